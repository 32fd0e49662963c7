// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 computes one 256 x 256 output tile per
// cluster of two CTAs (each CTA owns 128 rows of A, 128 of the 256 B rows, and the 128 x 256
// half of the accumulator that lands in its own TMEM). Sharing B across the pair halves the
// shared-memory traffic per FLOP, which is what bounds the single-CTA kernel in gemm.cu
// (operand reads plus TMA writes exceed 128 B/clk/SM at full tensor rate).
//
// Roles per CTA (6 warps): warp 0 TMA producer (loads its own A rows and its half of B into
// its own shared memory; both CTAs' loads complete on the LEADER's "full" barrier), warp 1
// MMA issuer (leader CTA only; both CTAs' warp 1 take part in the paired TMEM allocation),
// warps 2-5 epilogue (each CTA drains its own accumulator half). Barriers that must be seen
// by both CTAs are signalled twice (own address and the peer's address obtained with
// mapa), so no multicast form of any instruction is used. TMA loads are plain per-CTA loads.
//
// Same operand layouts, addend and rotary epilogues as gemm.cu; no split-K and no fused
// collectives here (those stay on the single-CTA kernel).
#include <algorithm>
#include <cstdio>

#include "common.cuh"

using namespace gfs;

namespace {

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BNH = 128;       // B rows (output columns) held per CTA
constexpr int BN = 256;        // output columns per tile
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;     // 16 KB
constexpr int B_BYTES = BNH * BK * 2;    // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 4 * 4096;
constexpr int SMEM_TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 256 + 1024;

struct Params2 {
  int M, N, K;
  int ldc, ldr;
  __nv_bfloat16* C;
  const __nv_bfloat16* R;  // addend (may alias C) or null
  int tiles_m, tiles_n, kblocks;
  uint32_t* status;
  const float* rope_cos;
  const float* rope_sin;
  int rope_cols, rope_d, rope_b;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D TMA load into this CTA's shared memory whose completion is counted on a barrier that may
// live in the peer CTA (cluster address). No multicast: every CTA fetches its own tiles.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once) on the barrier at `cluster_addr` when all MMAs issued so far by this thread are done
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const Params2 p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES]  (used in the leader)
  uint64_t* empty_bar = bars + STAGES;            // [STAGES]  (one per CTA)
  uint64_t* tmem_full = bars + 2 * STAGES;        // [2]       (one per CTA)
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;   // [2]       (used in the leader, 8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs initialised, TMEM allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  const int num_pairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;
  const int total_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < total_tiles; t += num_pairs) {
        const int m0 = (t / p.tiles_n) * 256 + static_cast<int>(rank) * BM;
        const int n0 = (t % p.tiles_n) * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tmap_a, bar, m0 + 64 * i, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BNH / 64; ++i) tma_load_2d_pair(sb + i * 8192, &tmap_b, bar, n0 + 64 * i, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) ------------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = pair; t < total_tiles; t += num_pairs) {
        mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, wctx, STATUS_TIMEOUT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          mbar_wait(&full_bar[stage], phase, wctx, STATUS_TIMEOUT_PIPE_FULL);
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // free this stage in both CTAs once the MMAs above have read it
          umma_commit_pair(mapa_u32(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(mapa_u32(smem_u32(&empty_bar[stage]), 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        umma_commit_pair(mapa_u32(smem_u32(&tmem_full[acc]), 0));
        umma_commit_pair(mapa_u32(smem_u32(&tmem_full[acc]), 1));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs, own accumulator half) ------------------------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint8_t* ebuf = epi_smem + (warp - 2) * 4096;
    const int rrow = lane >> 3;
    const int rch = lane & 7;
    const bool has_add = (p.R != nullptr);
    for (int t = pair; t < total_tiles; t += num_pairs) {
      const int m0 = (t / p.tiles_n) * 256 + static_cast<int>(rank) * BM;
      const int n0 = (t % p.tiles_n) * BN;
      mbar_wait(&tmem_full[acc], acc_phase, wctx, STATUS_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 64) {
        const int col0 = n0 + c;
        if (col0 >= p.N) break;
        const int gcol = col0 + rch * 8;
        uint4 pre[8];
        if (has_add) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int grow = m0 + q * 32 + i * 4 + rrow;
            pre[i] = make_uint4(0, 0, 0, 0);
            if (grow < p.M && gcol + 8 <= p.N)
              pre[i] = *reinterpret_cast<const uint4*>(p.R + static_cast<size_t>(grow) * p.ldr + gcol);
          }
        }
        uint32_t va[32], vb[32];
        tmem_ld_32x32(t_row + c, va);
        tmem_ld_32x32(t_row + c + 32, vb);
        tmem_ld_wait();
        uint8_t* myrow = ebuf + lane * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(va[8 * j + 0]), __uint_as_float(va[8 * j + 1]));
          w.y = pack_bf16x2(__uint_as_float(va[8 * j + 2]), __uint_as_float(va[8 * j + 3]));
          w.z = pack_bf16x2(__uint_as_float(va[8 * j + 4]), __uint_as_float(va[8 * j + 5]));
          w.w = pack_bf16x2(__uint_as_float(va[8 * j + 6]), __uint_as_float(va[8 * j + 7]));
          *reinterpret_cast<uint4*>(myrow + ((j ^ (lane & 7)) << 4)) = w;
          w.x = pack_bf16x2(__uint_as_float(vb[8 * j + 0]), __uint_as_float(vb[8 * j + 1]));
          w.y = pack_bf16x2(__uint_as_float(vb[8 * j + 2]), __uint_as_float(vb[8 * j + 3]));
          w.z = pack_bf16x2(__uint_as_float(vb[8 * j + 4]), __uint_as_float(vb[8 * j + 5]));
          w.w = pack_bf16x2(__uint_as_float(vb[8 * j + 6]), __uint_as_float(vb[8 * j + 7]));
          *reinterpret_cast<uint4*>(myrow + (((4 + j) ^ (lane & 7)) << 4)) = w;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + rrow;
          const int grow = m0 + q * 32 + r;
          uint4 w = *reinterpret_cast<const uint4*>(ebuf + r * 128 + ((rch ^ (r & 7)) << 4));
          if (grow < p.M && gcol + 8 <= p.N) {
            if (has_add || p.rope_cos != nullptr) {
              float f[8];
              const float2 x0 = unpack_bf16x2(w.x), x1 = unpack_bf16x2(w.y), x2 = unpack_bf16x2(w.z),
                           x3 = unpack_bf16x2(w.w);
              f[0] = x0.x; f[1] = x0.y; f[2] = x1.x; f[3] = x1.y; f[4] = x2.x; f[5] = x2.y; f[6] = x3.x; f[7] = x3.y;
              if (p.rope_cos != nullptr && gcol < p.rope_cols) {
                const int half = p.rope_d >> 1;
                const size_t ti = static_cast<size_t>(grow / p.rope_b) * half + ((gcol % p.rope_d) >> 1);
                const float4 cs = *reinterpret_cast<const float4*>(p.rope_cos + ti);
                const float4 sn = *reinterpret_cast<const float4*>(p.rope_sin + ti);
                const float a0 = f[0], a1 = f[1], a2 = f[2], a3 = f[3], a4 = f[4], a5 = f[5], a6 = f[6], a7 = f[7];
                f[0] = a0 * cs.x - a1 * sn.x; f[1] = a0 * sn.x + a1 * cs.x;
                f[2] = a2 * cs.y - a3 * sn.y; f[3] = a2 * sn.y + a3 * cs.y;
                f[4] = a4 * cs.z - a5 * sn.z; f[5] = a4 * sn.z + a5 * cs.z;
                f[6] = a6 * cs.w - a7 * sn.w; f[7] = a6 * sn.w + a7 * cs.w;
              }
              if (has_add) {
                const uint4 rr = pre[i];
                const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y), r2 = unpack_bf16x2(rr.z),
                             r3 = unpack_bf16x2(rr.w);
                f[0] += r0.x; f[1] += r0.y; f[2] += r1.x; f[3] += r1.y;
                f[4] += r2.x; f[5] += r2.y; f[6] += r3.x; f[7] += r3.y;
              }
              w.x = pack_bf16x2(f[0], f[1]);
              w.y = pack_bf16x2(f[2], f[3]);
              w.z = pack_bf16x2(f[4], f[5]);
              w.w = pack_bf16x2(f[6], f[7]);
            }
            *reinterpret_cast<uint4*>(p.C + static_cast<size_t>(grow) * p.ldc + gcol) = w;
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      // the accumulator buffer may be overwritten once all 8 epilogue warps of the pair are done
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // nobody leaves while the partner may still touch this CTA's shared memory / barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

template <bool A_MN, bool B_MN>
int launch2(const CUtensorMap* ta, const CUtensorMap* tb, const Params2& p, int grid, cudaStream_t stream) {
  auto kern = gemm2_kernel<A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) != cudaSuccess)
      return -10;
    attr_set = true;
  }
  kern<<<grid, THREADS, SMEM_TOTAL, stream>>>(*ta, *tb, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace

extern "C" {

// C[M,N] = op(A) op(B) (+R) on CTA pairs. Same conventions as gfs_gemm_bf16; intended for
// problems with at least one full wave of 256 x 256 tiles. Returns a negative value when the
// problem cannot be served (the caller then uses the single-CTA kernel).
int gfs_gemm2_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc,
                   int ldr, int a_mn_major, int b_mn_major, const void* rope_cos, const void* rope_sin, int rope_cols,
                   int rope_d, int rope_b, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || (R && (ldr & 7))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(R)) & 15)
    return -2;
  const CUtensorMap* ta = a_mn_major ? gfs_host::tmap_2d_cached(A, K, M, lda, 64, 64)
                                     : gfs_host::tmap_2d_cached(A, M, K, lda, BM, 64);
  const CUtensorMap* tb = b_mn_major ? gfs_host::tmap_2d_cached(B, K, N, ldb, 64, 64)
                                     : gfs_host::tmap_2d_cached(B, N, K, ldb, BNH, 64);
  if (ta == nullptr || tb == nullptr) return -3;
  Params2 p{};
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (N + BN - 1) / BN;
  p.kblocks = (K + BK - 1) / BK;
  p.status = gfs_host::status_words();
  p.rope_cos = static_cast<const float*>(rope_cos);
  p.rope_sin = static_cast<const float*>(rope_sin);
  p.rope_cols = rope_cols; p.rope_d = rope_d; p.rope_b = rope_b > 0 ? rope_b : 1;
  const int pairs = std::min(p.tiles_m * p.tiles_n, gfs_host::sm_count() / 2);
  const int grid = 2 * pairs;
  if (!a_mn_major && !b_mn_major) return launch2<false, false>(ta, tb, p, grid, stream);
  if (!a_mn_major && b_mn_major) return launch2<false, true>(ta, tb, p, grid, stream);
  if (a_mn_major && b_mn_major) return launch2<true, true>(ta, tb, p, grid, stream);
  return launch2<true, false>(ta, tb, p, grid, stream);
}

}  // extern "C"
