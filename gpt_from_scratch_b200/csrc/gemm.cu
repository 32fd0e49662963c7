// bf16 GEMM for sm_100a: C[M,N] = op(A)[M,K] * op(B)[K,N] (+ R), fp32 accumulation in TMEM.
//
// One persistent CTA per SM, six warps with fixed roles:
//   warp 0    TMA producer  (cp.async.bulk.tensor 2-D loads, 128-byte swizzle, STAGES-deep ring)
//   warp 1    MMA issuer    (one thread issues tcgen05.mma 128xBNx16; owns the TMEM allocation)
//   warps 2-5 epilogue      (tcgen05.ld -> registers -> bf16/fp32 global stores), double-buffered
//                           accumulators so tile i's epilogue overlaps tile i+1's main loop
//
// Operand layouts (all row-major in global memory, leading dimension in elements):
//   A K-major : A is [M, K]          A MN-major: A is stored as [K, M]
//   B K-major : B is [N, K]          B MN-major: B is stored as [K, N]
// which covers the three GEMMs of a linear layer without any transposed copies:
//   forward  Y = X W^T        : A = X  (K-major),  B = W  (K-major)
//   dgrad    dX = dY W        : A = dY (K-major),  B = W  (MN-major, contraction over W's rows)
//   wgrad    dW = dY^T X      : A = dY (MN-major), B = X  (MN-major), contraction over tokens
//
// Small outputs (wgrad of the per-layer linears) use deterministic split-K: each split
// writes an fp32 partial tile to a workspace and a second kernel sums the splits in a
// fixed order, adds the optional addend and rounds once to bf16.
//
// Counterpart in the reference: the cuBLAS calls behind F.linear and its autograd
// (core/tensor_parallel/layers.py:47,82).
#include <algorithm>
#include <cstdio>

#include "common.cuh"

using namespace gfs;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int COMM_THREADS = 64;        // two extra warps in the fused-collective variants
constexpr int MAX_PEERS = 8;

enum CommMode : int { COMM_NONE = 0, COMM_ALLGATHER = 1, COMM_REDUCE_SCATTER = 2 };

// Arguments of the fused collective (all-gather of A's rows before the product, or
// reduce-scatter of the product's rows after it) over peer memory.
struct CommParams {
  int world, rank;
  int rows_per_rank;                    // rows of the sharded dimension per rank (multiple of BM)
  // all-gather: the local shard is pushed into every rank's gathered buffer
  const __nv_bfloat16* ag_src;          // [rows_per_rank, ag_cols], pitch ag_ld
  int ag_ld, ag_cols;
  __nv_bfloat16* peer_buf[MAX_PEERS];   // AG: gathered [world*rows_per_rank, ag_cols]; RS: staging [world][rows_per_rank][N]
  // reduce-scatter: out[rows_per_rank, N] = sum over ranks of their partial rows (+ residual)
  __nv_bfloat16* rs_out;
  const __nv_bfloat16* rs_res;
  int rs_ld_out, rs_ld_res;
  __nv_bfloat16* mc_buf;                // all-gather: multicast address of the gathered buffers, or null
  uint32_t* peer_flags[MAX_PEERS];      // flags[p][src]: progress of rank src's writes into rank p
  uint32_t target;                      // value flags[rank][src] must reach in this call
  unsigned long long wait_ns;
};

enum EpiMode : int { EPI_STORE = 0, EPI_ADD = 1, EPI_PARTIAL_F32 = 2 };

struct GemmParams {
  int M, N, K;
  int ldc, ldr;
  __nv_bfloat16* C;
  const __nv_bfloat16* R;
  float* ws;
  int split_k;
  int kblocks_total;
  int kblocks_per_split;
  int tiles_m, tiles_n;
  int epi_mode;
  uint32_t* status;
  // optional rotary embedding applied to the first rope_cols output columns (interleaved
  // pairs inside heads of rope_d columns); output row r belongs to position r / rope_b
  const float* rope_cos;
  const float* rope_sin;
  int rope_cols, rope_d, rope_b;
  // SwiGLU fusion. mode 1 (forward, B = [gate rows | up rows] of a [2I, K] weight): each tile
  // pairs 128 gate columns with the matching 128 up columns; the epilogue writes both halves
  // of the projection (C, pitch ldc) and act = silu(gate) * up (swi_act, pitch swi_ld).
  // mode 2 (backward, the product is d_act [M, I]): the epilogue reads gate/up from swi_gu
  // (pitch swi_ld) and writes d_gate | d_up into C ([M, 2I], pitch ldc) instead of d_act.
  int swi_mode, swi_I, swi_ld;
  __nv_bfloat16* swi_act;
  const __nv_bfloat16* swi_gu;
  CommParams comm;
};

__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// Tile order. Plain: n fastest. Fused collectives walk the row chunks of the ranks in a
// rotated order: all-gather starts with the local chunk (already in place), reduce-scatter
// ends with it (its rows need no transfer), so remote traffic overlaps the other chunks' math.
template <int BN, int COMM>
__device__ __forceinline__ void decode_tile(const GemmParams& p, int t, int& z, int& m0, int& n0, int& chunk) {
  if (COMM == COMM_NONE) {
    const int tiles_mn = p.tiles_m * p.tiles_n;
    z = t / tiles_mn;
    const int mn = t - z * tiles_mn;
    m0 = (mn / p.tiles_n) * BM;
    n0 = (mn % p.tiles_n) * BN;
    chunk = 0;
  } else {
    const int tiles_per_chunk = (p.comm.rows_per_rank / BM) * p.tiles_n;
    const int ci = t / tiles_per_chunk;
    const int rem = t - ci * tiles_per_chunk;
    chunk = (p.comm.rank + ci + (COMM == COMM_REDUCE_SCATTER ? 1 : 0)) % p.comm.world;
    z = 0;
    m0 = chunk * p.comm.rows_per_rank + (rem / p.tiles_n) * BM;
    n0 = (rem % p.tiles_n) * BN;
  }
}

template <int BN, int STAGES>
struct SmemCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int EPI_BYTES = 4 * 4096;  // one [32 rows x 128 B] transpose buffer per epilogue warp
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;  // + slack for 1024-B alignment
};

template <bool A_MN, bool B_MN, int BN, int STAGES, int COMM>
__global__ void __launch_bounds__(GEMM_THREADS + (COMM != COMM_NONE ? COMM_THREADS : 0), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using Cfg = SmemCfg<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle wants tile bases aligned to 1024 B.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* epi_smem = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::EPI_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES]
  uint64_t* empty_bar = bars + STAGES;        // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;    // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();       // set-up above may overlap the tail of the preceding kernel (programmatic launch)
  pdl_trigger();
  const uint32_t tmem_base = *tmem_base_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  const int tiles_mn = p.tiles_m * p.tiles_n;
  const int total_tiles = tiles_mn * p.split_k;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t chunk_ready = 0;  // all-gather: chunks whose arrival has been observed
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        int z, m0, n0, chunk;
        decode_tile<BN, COMM>(p, t, z, m0, n0, chunk);
        if (COMM == COMM_ALLGATHER && !((chunk_ready >> chunk) & 1u)) {
          // rows of this chunk are written into our gathered buffer by rank `chunk`
          if (!*abort_flag &&
              !wait_flag_reached(p.comm.peer_flags[p.comm.rank] + chunk, p.comm.target, p.comm.wait_ns, p.status,
                                 0xA6000000u | (chunk << 8) | p.comm.rank))
            *abort_flag = 1u;
          fence_proxy_async_global();  // peer's generic-proxy stores -> our TMA (async proxy) loads
          chunk_ready |= 1u << chunk;
        }
        const int kb0 = z * p.kblocks_per_split;
        const int kb1 = min(p.kblocks_total, kb0 + p.kblocks_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
          uint8_t* sa = tiles + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, &tmap_a, &full_bar[stage], m0 + 64 * i, k0);
          }
          if (!B_MN) {
            if (p.swi_mode == 1) {  // 128 gate rows + the matching 128 up rows (tensor map box = 128 rows)
              tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0 >> 1);
              tma_load_2d(sb + (BN / 2) * 128, &tmap_b, &full_bar[stage], k0, p.swi_I + (n0 >> 1));
            } else {
              tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
            }
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmap_b, &full_bar[stage], n0 + 64 * i, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_flag) {
        // let copies that are still in flight land before the CTA's shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    {  // whole warp, converged: the MMA / commit helpers elect the issuing lane
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        const int z = (COMM == COMM_NONE) ? t / tiles_mn : 0;
        const int kb0 = z * p.kblocks_per_split;
        const int kb1 = min(p.kblocks_total, kb0 + p.kblocks_per_split);
        mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, wctx, STATUS_TIMEOUT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&full_bar[stage], phase, wctx, STATUS_TIMEOUT_PIPE_FULL);
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + k * 2048, 8192, 1024)
                                        : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_ss_e(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_e(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        umma_commit_e(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    // all-gather variant: until the first accumulator is ready these warps help the two push warps
    if (COMM == COMM_ALLGATHER) ag_push_rows(p.comm, static_cast<int>(threadIdx.x) - 64, COMM_THREADS + 128, 1);
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      int z, m0, n0, chunk;
      decode_tile<BN, COMM>(p, t, z, m0, n0, chunk);
      mbar_wait(&tmem_full[acc], acc_phase, wctx, STATUS_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (p.epi_mode == EPI_PARTIAL_F32) {
        // split-K partial tile: fp32 rows straight to the workspace
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int col0 = n0 + c;
          if (col0 >= p.N) break;
          uint32_t v[32];
          tmem_ld_32x32(t_row + c, v);
          tmem_ld_wait();
          if (row < p.M) {
            float* dst = p.ws + (static_cast<size_t>(z) * p.M + row) * p.N + col0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (col0 + 4 * j + 4 <= p.N) {
                float4 o = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                *reinterpret_cast<float4*>(dst + 4 * j) = o;
              }
            }
          }
        }
      } else if (p.swi_mode == 1) {
        // SwiGLU forward: accumulator columns [0,128) are gate, [128,256) the matching up columns
        uint8_t* ebuf = epi_smem + (warp - 2) * 4096;
        const int g0 = n0 >> 1;  // first gate column of the tile
        const int rrow = lane >> 3;
        const int rch = lane & 7;
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          if (g0 + c >= p.swi_I) break;
          uint32_t vg[32], vu[32];
          tmem_ld_32x32(t_row + c, vg);
          tmem_ld_32x32(t_row + BN / 2 + c, vu);
          tmem_ld_wait();
          uint32_t pa[16];
          uint8_t* myrow = ebuf + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 wg, wu;
            uint32_t* wgp = &wg.x;
            uint32_t* wup = &wu.x;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              wgp[e] = pack_bf16x2(__uint_as_float(vg[8 * j + 2 * e]), __uint_as_float(vg[8 * j + 2 * e + 1]));
              wup[e] = pack_bf16x2(__uint_as_float(vu[8 * j + 2 * e]), __uint_as_float(vu[8 * j + 2 * e + 1]));
              // act from the bf16-rounded projections, silu rounded to bf16 before the product
              const float2 g2 = unpack_bf16x2(wgp[e]), u2 = unpack_bf16x2(wup[e]);
              const float s0 = __bfloat162float(__float2bfloat16_rn(g2.x * sigmoid_f(g2.x)));
              const float s1 = __bfloat162float(__float2bfloat16_rn(g2.y * sigmoid_f(g2.y)));
              pa[4 * j + e] = pack_bf16x2(s0 * u2.x, s1 * u2.y);
            }
            *reinterpret_cast<uint4*>(myrow + ((j ^ (lane & 7)) << 4)) = wg;
            *reinterpret_cast<uint4*>(myrow + (((4 + j) ^ (lane & 7)) << 4)) = wu;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {  // gate | up halves of the projection
            const int r = i * 4 + rrow;
            const int grow = m0 + q * 32 + r;
            const int lc = g0 + c + (rch & 3) * 8;  // column inside [0, I)
            const uint4 w = *reinterpret_cast<const uint4*>(ebuf + r * 128 + ((rch ^ (r & 7)) << 4));
            if (grow < p.M && lc + 8 <= p.swi_I)
              *reinterpret_cast<uint4*>(p.C + static_cast<size_t>(grow) * p.ldc + (rch >= 4 ? p.swi_I : 0) + lc) = w;
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(myrow + ((j ^ (lane & 7)) << 4)) =
                make_uint4(pa[4 * j], pa[4 * j + 1], pa[4 * j + 2], pa[4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {  // act: 32 columns per row, 4 lanes per row
            const int r = i * 8 + (lane >> 2);
            const int ch = lane & 3;
            const int grow = m0 + q * 32 + r;
            const int lc = g0 + c + ch * 8;
            const uint4 w = *reinterpret_cast<const uint4*>(ebuf + r * 128 + ((ch ^ (r & 7)) << 4));
            if (grow < p.M && lc + 8 <= p.swi_I)
              *reinterpret_cast<uint4*>(p.swi_act + static_cast<size_t>(grow) * p.swi_ld + lc) = w;
          }
          __syncwarp();
        }
      } else {
        // bf16 output. Each lane owns one accumulator row; a per-warp shared-memory transpose
        // turns that into stores where 8 lanes write one full 128-byte line of a row
        // (row-per-lane stores would touch 32 different lines per instruction). Rotary
        // embedding and the addend are applied after the transpose on 8-column groups.
        uint8_t* ebuf = epi_smem + (warp - 2) * 4096;
        const int rrow = lane >> 3;
        const int rch = lane & 7;
        const bool has_math = (p.epi_mode == EPI_ADD) || (p.rope_cos != nullptr);
        const bool swi_bwd = (p.swi_mode == 2);
#pragma unroll 1
        for (int c = 0; c < BN; c += 64) {
          const int col0 = n0 + c;
          if (col0 >= p.N) break;
          const int gcol = col0 + rch * 8;
          // the addend (and, in the SwiGLU backward, gate/up) are fetched up front: issued
          // after the stores below they would be serialised behind them (the addend may alias C)
          uint4 pre0[8], pre1[8];
          if (p.epi_mode == EPI_ADD || swi_bwd) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int grow = m0 + q * 32 + i * 4 + rrow;
              pre0[i] = make_uint4(0, 0, 0, 0);
              pre1[i] = make_uint4(0, 0, 0, 0);
              if (grow < p.M && gcol + 8 <= p.N) {
                if (swi_bwd) {
                  const __nv_bfloat16* gp = p.swi_gu + static_cast<size_t>(grow) * p.swi_ld + gcol;
                  pre0[i] = *reinterpret_cast<const uint4*>(gp);
                  pre1[i] = *reinterpret_cast<const uint4*>(gp + p.swi_I);
                } else {
                  pre0[i] = *reinterpret_cast<const uint4*>(p.R + static_cast<size_t>(grow) * p.ldr + gcol);
                }
              }
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
            if (swi_bwd) {
              // w holds 8 values of d_act; turn them into d_gate and d_up
              if (grow < p.M && gcol + 8 <= p.N) {
                const uint4 gq = pre0[i];
                const uint4 uq = pre1[i];
                const uint32_t* dw = &w.x;
                const uint32_t* gw = &gq.x;
                const uint32_t* uw = &uq.x;
                uint4 og, ou;
                uint32_t* ogp = &og.x;
                uint32_t* oup = &ou.x;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 d2 = unpack_bf16x2(dw[e]), g2 = unpack_bf16x2(gw[e]), u2 = unpack_bf16x2(uw[e]);
                  const float sg0 = sigmoid_f(g2.x), sg1 = sigmoid_f(g2.y);
                  ogp[e] = pack_bf16x2(d2.x * u2.x * sg0 * (1.f + g2.x * (1.f - sg0)),
                                       d2.y * u2.y * sg1 * (1.f + g2.y * (1.f - sg1)));
                  oup[e] = pack_bf16x2(d2.x * g2.x * sg0, d2.y * g2.y * sg1);
                }
                __nv_bfloat16* dst = p.C + static_cast<size_t>(grow) * p.ldc + gcol;
                *reinterpret_cast<uint4*>(dst) = og;
                *reinterpret_cast<uint4*>(dst + p.swi_I) = ou;
              }
            } else if (grow < p.M && gcol + 8 <= p.N) {
              if (has_math) {
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
                if (p.epi_mode == EPI_ADD) {
                  const uint4 rr = pre0[i];
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
              __nv_bfloat16* dst;
              if (COMM == COMM_REDUCE_SCATTER) {
                // partial rows go to their owner's staging area, slot of this (source) rank
                dst = p.comm.peer_buf[chunk] +
                      (static_cast<size_t>(p.comm.rank) * p.comm.rows_per_rank +
                       (grow - chunk * p.comm.rows_per_rank)) * p.N + gcol;
              } else {
                dst = p.C + static_cast<size_t>(grow) * p.ldc + gcol;
              }
              *reinterpret_cast<uint4*>(dst) = w;
            }
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();  // orders every lane's (peer) stores before lane 0's release below
      if (lane == 0) {
        mbar_arrive(&tmem_empty[acc]);
        if (COMM == COMM_REDUCE_SCATTER) red_release_sys_add_u32(p.comm.peer_flags[chunk] + p.comm.rank, 1u);
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (COMM == COMM_REDUCE_SCATTER) {
      // tiles done: join the reduction of this rank's row chunk (second share of the vectors)
      const CommParams& c = p.comm;
      bool ok = true;
      for (int src = 0; src < c.world; ++src)
        ok = wait_flag_reached(c.peer_flags[c.rank] + src, c.target, c.wait_ns, p.status,
                               0xB6000000u | (src << 8) | c.rank) && ok;
      if (!ok) *abort_flag = 1u;
      constexpr int RED_THREADS = COMM_THREADS + 128;
      rs_reduce_rows(c.peer_buf[c.rank], c.world, c.rows_per_rank, p.N, c.rs_res, c.rs_ld_res, c.rs_out, c.rs_ld_out,
                     static_cast<size_t>(blockIdx.x) * RED_THREADS + COMM_THREADS + (threadIdx.x - 64),
                     static_cast<size_t>(gridDim.x) * RED_THREADS);
    }
  } else if (COMM == COMM_ALLGATHER) {
    // ------------------------------ all-gather push (warps 6-7) ------------------------------
    // Every CTA pushes its slice of the local shard into every rank's gathered buffer
    // (own rank first), then bumps that rank's counter for this source.
    // (the epilogue warps push too, before their first tile: see the top of the epilogue branch)
    ag_push_rows(p.comm, static_cast<int>(threadIdx.x) - GEMM_THREADS + 128, COMM_THREADS + 128, 1);
  } else if (COMM == COMM_REDUCE_SCATTER) {
    // ------------------------------ reduce (warps 6-7) ------------------------------
    // Wait until every rank (this one included) has delivered all partial tiles of our row
    // chunk, then sum the staged partials in rank order, add the residual, round once.
    const CommParams& c = p.comm;
    const int ct = threadIdx.x - GEMM_THREADS;
    bool ok = true;
    for (int src = 0; src < c.world; ++src)
      ok = wait_flag_reached(c.peer_flags[c.rank] + src, c.target, c.wait_ns, p.status,
                             0xB5000000u | (src << 8) | c.rank) && ok;
    if (!ok) *abort_flag = 1u;
    // these 64 threads take the first share of the vectors; the epilogue warps take the rest once
    // their tiles are done (see the end of the epilogue loop)
    constexpr int RED_THREADS = COMM_THREADS + 128;
    rs_reduce_rows(c.peer_buf[c.rank], c.world, c.rows_per_rank, p.N, c.rs_res, c.rs_ld_res, c.rs_out, c.rs_ld_out,
                   static_cast<size_t>(blockIdx.x) * RED_THREADS + ct, static_cast<size_t>(gridDim.x) * RED_THREADS);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// Sum split-K partials in split order, add the optional addend, round once to bf16.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ C,
                                     const __nv_bfloat16* __restrict__ R, int M, int N, int ldc, int ldr, int splits,
                                     int add) {
  const int groups_per_row = N >> 3;
  const size_t total = static_cast<size_t>(M) * groups_per_row;
  for (size_t g = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; g < total;
       g += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(g / groups_per_row);
    const int col = static_cast<int>(g % groups_per_row) << 3;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int z = 0; z < splits; ++z) {
      const float4* src = reinterpret_cast<const float4*>(ws + (static_cast<size_t>(z) * M + row) * N + col);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    if (add) {
      const uint4 rr = *reinterpret_cast<const uint4*>(R + static_cast<size_t>(row) * ldr + col);
      const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y), r2 = unpack_bf16x2(rr.z),
                   r3 = unpack_bf16x2(rr.w);
      acc[0] += r0.x; acc[1] += r0.y; acc[2] += r1.x; acc[3] += r1.y;
      acc[4] += r2.x; acc[5] += r2.y; acc[6] += r3.x; acc[7] += r3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(C + static_cast<size_t>(row) * ldc + col) = o;
  }
}

template <bool A_MN, bool B_MN, int BN, int STAGES, int COMM = COMM_NONE>
int launch_variant(const CUtensorMap* ta, const CUtensorMap* tb, const GemmParams& p, int grid, cudaStream_t stream) {
  using Cfg = SmemCfg<BN, STAGES>;
  auto kern = gemm_bf16_kernel<A_MN, B_MN, BN, STAGES, COMM>;
  static bool attr_set = false;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set || attr_dev != dev) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::TOTAL) != cudaSuccess) return -10;
    attr_set = true;
    attr_dev = dev;
  }
  if (gfs_host::launch_pdl(kern, dim3(grid), dim3(GEMM_THREADS + (COMM != COMM_NONE ? COMM_THREADS : 0)), Cfg::TOTAL,
                           stream, *ta, *tb, p) != cudaSuccess)
    return -11;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int choose_split(int tiles, int kblocks, int sms, size_t mn_elems, size_t ws_bytes) {
  if (tiles * 10 >= sms * 9 || kblocks < 8) return 1;
  int best = 1;
  long best_cost = 1L << 60;
  for (int s = 1; s <= 16; ++s) {
    const int per = (kblocks + s - 1) / s;
    if (per < 4) break;
    if ((per * (s - 1)) >= kblocks) continue;  // would leave an empty split
    if (s > 1 && static_cast<size_t>(s) * mn_elems * 4 > ws_bytes) break;
    const long waves = (static_cast<long>(tiles) * s + sms - 1) / sms;
    const long cost = waves * (per + 6) + (s > 1 ? 6 * s : 0);
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

}  // namespace

extern "C" {

// C[M,N] = op(A) op(B) (+R when add != 0). See the file header for operand layouts.
// ws/ws_bytes: fp32 workspace for split-K (may be null: split-K is then disabled).
// force_split: 0 = automatic, >0 = use exactly that many splits (tests).
// Returns 0 on success, a negative value if the arguments cannot be served.
int gfs_gemm_bf16_rope(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                       int ldc, int ldr, int a_mn_major, int b_mn_major, int add, void* ws, size_t ws_bytes,
                       int force_split, const void* rope_cos, const void* rope_sin, int rope_cols, int rope_d,
                       int rope_b, void* stream_);

int gfs_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc,
                  int ldr, int a_mn_major, int b_mn_major, int add, void* ws, size_t ws_bytes, int force_split,
                  void* stream_) {
  return gfs_gemm_bf16_rope(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn_major, b_mn_major, add, ws, ws_bytes,
                            force_split, nullptr, nullptr, 0, 0, 1, stream_);
}

// Same product with a rotary-embedding epilogue: the first rope_cols output columns are
// rotated pairwise with cos/sin[row / rope_b][(col % rope_d) / 2] (fp32 tables [positions, rope_d/2]).
// Split-K is disabled when the rotation is requested.
int gfs_gemm_bf16_rope(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                       int ldc, int ldr, int a_mn_major, int b_mn_major, int add, void* ws, size_t ws_bytes,
                       int force_split, const void* rope_cos, const void* rope_sin, int rope_cols, int rope_d,
                       int rope_b, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rope_cos != nullptr) {
    if ((rope_d & 7) || (rope_cols & 7) || rope_b <= 0) return -1;
    ws = nullptr;
  }
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || (add && (ldr & 7))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       (add ? reinterpret_cast<uintptr_t>(R) : 0)) & 15)
    return -2;
  const int BN = (N > 128) ? 256 : 128;
  const CUtensorMap* ta = a_mn_major ? gfs_host::tmap_2d_cached(A, K, M, lda, 64, 64)
                                     : gfs_host::tmap_2d_cached(A, M, K, lda, BM, 64);
  const CUtensorMap* tb = b_mn_major ? gfs_host::tmap_2d_cached(B, K, N, ldb, 64, 64)
                                     : gfs_host::tmap_2d_cached(B, N, K, ldb, BN, 64);
  if (ta == nullptr || tb == nullptr) return -3;

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ws = static_cast<float*>(ws);
  p.rope_cos = static_cast<const float*>(rope_cos);
  p.rope_sin = static_cast<const float*>(rope_sin);
  p.rope_cols = rope_cols; p.rope_d = rope_d; p.rope_b = rope_b;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.kblocks_total = (K + BK - 1) / BK;
  p.status = gfs_host::status_words();
  const int sms = gfs_host::sm_count();
  const int tiles = p.tiles_m * p.tiles_n;
  int split = 1;
  if (ws != nullptr) {
    split = force_split > 0 ? force_split
                            : choose_split(tiles, p.kblocks_total, sms, static_cast<size_t>(M) * N, ws_bytes);
    if (split > p.kblocks_total) split = p.kblocks_total;
    if (split > 1 && static_cast<size_t>(split) * M * N * 4 > ws_bytes) split = 1;
  }
  p.kblocks_per_split = (p.kblocks_total + split - 1) / split;
  split = (p.kblocks_total + p.kblocks_per_split - 1) / p.kblocks_per_split;  // no empty splits
  p.split_k = split;
  p.epi_mode = split > 1 ? EPI_PARTIAL_F32 : (add ? EPI_ADD : EPI_STORE);
  const int grid = std::min(tiles * split, sms);

  int rc;
  if (BN == 256) {
    if (!a_mn_major && !b_mn_major) rc = launch_variant<false, false, 256, 4>(ta, tb, p, grid, stream);
    else if (!a_mn_major && b_mn_major) rc = launch_variant<false, true, 256, 4>(ta, tb, p, grid, stream);
    else if (a_mn_major && b_mn_major) rc = launch_variant<true, true, 256, 4>(ta, tb, p, grid, stream);
    else rc = launch_variant<true, false, 256, 4>(ta, tb, p, grid, stream);
  } else {
    if (!a_mn_major && !b_mn_major) rc = launch_variant<false, false, 128, 6>(ta, tb, p, grid, stream);
    else if (!a_mn_major && b_mn_major) rc = launch_variant<false, true, 128, 6>(ta, tb, p, grid, stream);
    else if (a_mn_major && b_mn_major) rc = launch_variant<true, true, 128, 6>(ta, tb, p, grid, stream);
    else rc = launch_variant<true, false, 128, 6>(ta, tb, p, grid, stream);
  }
  if (rc != 0) return rc;
  if (split > 1) {
    const size_t groups = static_cast<size_t>(M) * (N >> 3);
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<size_t>((groups + threads - 1) / threads, static_cast<size_t>(sms) * 8));
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(p.ws, p.C, p.R, M, N, ldc, ldr, split, add);
    if (cudaGetLastError() != cudaSuccess) return -12;
  }
  return 0;
}

// SwiGLU-fused products of the MLP (see GemmParams::swi_mode).
//   mode 1: gu[M, 2I] = x[M, K] @ w_gu[2I, K]^T and act[M, I] = silu(gu[:, :I]) * gu[:, I:]
//           (a = x, b = w_gu, c = gu with pitch ldc, extra = act with pitch ld_extra)
//   mode 2: d_gu[M, 2I] = swiglu_backward(d_act = dy[M, K] @ w_down[K, I], gu)
//           (a = dy, b = w_down stored [K, I], c = d_gu with pitch ldc, extra = gu with pitch ld_extra)
int gfs_gemm_bf16_swiglu(int mode, const void* a, const void* b, void* c, void* extra, int M, int I, int K, int lda,
                         int ldb, int ldc, int ld_extra, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (mode != 1 && mode != 2) return -1;
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if ((I & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || (ld_extra & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
       reinterpret_cast<uintptr_t>(extra)) & 15)
    return -2;
  constexpr int BN = 256;
  GemmParams p{};
  p.M = M; p.K = K;
  p.N = (mode == 1) ? 2 * I : I;
  p.C = static_cast<__nv_bfloat16*>(c);
  p.ldc = ldc;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (mode == 1) ? (I + BN / 2 - 1) / (BN / 2) : (I + BN - 1) / BN;
  p.kblocks_total = (K + BK - 1) / BK;
  p.kblocks_per_split = p.kblocks_total;
  p.split_k = 1;
  p.epi_mode = EPI_STORE;
  p.status = gfs_host::status_words();
  p.rope_b = 1;
  p.swi_mode = mode;
  p.swi_I = I;
  p.swi_ld = ld_extra;
  if (mode == 1) p.swi_act = static_cast<__nv_bfloat16*>(extra);
  else p.swi_gu = static_cast<const __nv_bfloat16*>(extra);
  const CUtensorMap* ta = gfs_host::tmap_2d_cached(a, M, K, lda, BM, 64);
  const CUtensorMap* tb = (mode == 1) ? gfs_host::tmap_2d_cached(b, 2 * I, K, ldb, BN / 2, 64)
                                      : gfs_host::tmap_2d_cached(b, K, I, ldb, 64, 64);
  if (ta == nullptr || tb == nullptr) return -3;
  const int grid = std::min(p.tiles_m * p.tiles_n, gfs_host::sm_count());
  return (mode == 1) ? launch_variant<false, false, 256, 4>(ta, tb, p, grid, stream)
                     : launch_variant<false, true, 256, 4>(ta, tb, p, grid, stream);
}

// Fused collective + GEMM over peer memory (one kernel, no NCCL):
//   mode 1 (all-gather -> GEMM): `a` is this rank's shard [M/world, K]; every rank's kernel
//     pushes its shard into all gathered buffers (peer_bufs[p] = rank p's [M, K] buffer) while
//     its tensor cores already work on the chunks that have arrived; out = gathered @ op(B) -> [M, N].
//   mode 2 (GEMM -> reduce-scatter): `a` is the full [M, K] operand; partial output rows are
//     stored straight into their owner's staging area (peer_bufs[p] = rank p's [world, M/world, N])
//     and the owner sums them (+ residual) into out [M/world, N].
// peer_flags[p] = rank p's uint32 counters for this call site (>= world entries, zero at start,
// never reset); *target_inout is the cumulative value the counters must reach: the function
// advances it by this call's increment, identically on every rank.
// A is K-major; B is [N, K] or, with b_mn_major, [K, N]. M/world must be a multiple of 128.
int gfs_gemm_bf16_comm(int mode, const void* a, int lda, const void* B, int ldb, void* out, int ldo,
                       const void* residual, int ldr, int M, int N, int K, int b_mn_major, int world, int rank,
                       const unsigned long long* peer_bufs, const unsigned long long* peer_flags,
                       unsigned int* target_inout, const void* rope_cos, const void* rope_sin, int rope_cols,
                       int rope_d, int rope_b, long long wait_ns, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (mode != COMM_ALLGATHER && mode != COMM_REDUCE_SCATTER) return -1;
  if (world < 2 || world > MAX_PEERS || rank < 0 || rank >= world) return -1;
  if (M <= 0 || N <= 0 || K <= 0 || (M % world) != 0 || ((M / world) % BM) != 0) return -1;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldo & 7) || (residual && (ldr & 7))) return -1;
  const int rows_per_rank = M / world;
  const int BN = (N > 128) ? 256 : 128;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.kblocks_total = (K + BK - 1) / BK;
  p.kblocks_per_split = p.kblocks_total;
  p.split_k = 1;
  p.epi_mode = EPI_STORE;
  p.status = gfs_host::status_words();
  p.rope_cos = static_cast<const float*>(rope_cos);
  p.rope_sin = static_cast<const float*>(rope_sin);
  p.rope_cols = rope_cols; p.rope_d = rope_d; p.rope_b = rope_b > 0 ? rope_b : 1;
  CommParams& c = p.comm;
  c.world = world; c.rank = rank; c.rows_per_rank = rows_per_rank;
  c.wait_ns = wait_ns > 0 ? static_cast<unsigned long long>(wait_ns) : 20000000000ull;
  for (int i = 0; i < world; ++i) {
    c.peer_buf[i] = reinterpret_cast<__nv_bfloat16*>(peer_bufs[i]);
    c.peer_flags[i] = reinterpret_cast<uint32_t*>(peer_flags[i]);
  }
  // entry `world` of the buffer table: multicast address of the same buffers (0 = none). With two
  // ranks a multicast store saves nothing (one peer) and sends the local copy through the switch
  // as well (measured slower: 8.46 vs 8.28 ms per GPT-124M TP2 step), so it is used from 3 ranks up.
  c.mc_buf = (mode == COMM_ALLGATHER && world > 2) ? reinterpret_cast<__nv_bfloat16*>(peer_bufs[world]) : nullptr;
  const int sms = gfs_host::sm_count();
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = std::min(tiles, sms);
  const void* a_base;
  int a_ld;
  if (mode == COMM_ALLGATHER) {
    c.ag_src = static_cast<const __nv_bfloat16*>(a);
    c.ag_ld = lda;
    c.ag_cols = K;
    a_base = c.peer_buf[rank];   // the GEMM reads the local gathered buffer
    a_ld = K;
    p.C = static_cast<__nv_bfloat16*>(out);
    p.ldc = ldo;
    *target_inout += static_cast<unsigned int>(grid);   // every CTA of a source signals once per destination
  } else {
    a_base = a;
    a_ld = lda;
    c.rs_out = static_cast<__nv_bfloat16*>(out);
    c.rs_ld_out = ldo;
    c.rs_res = static_cast<const __nv_bfloat16*>(residual);
    c.rs_ld_res = ldr;
    *target_inout += static_cast<unsigned int>((rows_per_rank / BM) * p.tiles_n * 4);  // 4 epilogue warps per tile
  }
  c.target = *target_inout;
  if ((reinterpret_cast<uintptr_t>(a_base) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return -2;
  const CUtensorMap* ta = gfs_host::tmap_2d_cached(a_base, M, K, a_ld, BM, 64);
  const CUtensorMap* tb = b_mn_major ? gfs_host::tmap_2d_cached(B, K, N, ldb, 64, 64)
                                     : gfs_host::tmap_2d_cached(B, N, K, ldb, BN, 64);
  if (ta == nullptr || tb == nullptr) return -3;
  int rc;
  if (mode == COMM_ALLGATHER) {
    if (BN == 256) rc = b_mn_major ? launch_variant<false, true, 256, 4, COMM_ALLGATHER>(ta, tb, p, grid, stream)
                                   : launch_variant<false, false, 256, 4, COMM_ALLGATHER>(ta, tb, p, grid, stream);
    else rc = b_mn_major ? launch_variant<false, true, 128, 6, COMM_ALLGATHER>(ta, tb, p, grid, stream)
                         : launch_variant<false, false, 128, 6, COMM_ALLGATHER>(ta, tb, p, grid, stream);
  } else {
    if (BN == 256) rc = b_mn_major ? launch_variant<false, true, 256, 4, COMM_REDUCE_SCATTER>(ta, tb, p, grid, stream)
                                   : launch_variant<false, false, 256, 4, COMM_REDUCE_SCATTER>(ta, tb, p, grid, stream);
    else rc = b_mn_major ? launch_variant<false, true, 128, 6, COMM_REDUCE_SCATTER>(ta, tb, p, grid, stream)
                         : launch_variant<false, false, 128, 6, COMM_REDUCE_SCATTER>(ta, tb, p, grid, stream);
  }
  return rc;
}

// Number of kernels gfs_gemm_bf16 launches for this problem (1, or 2 with split-K).
int gfs_gemm_bf16_launches(int M, int N, int K, size_t ws_bytes) {
  const int BN = (N > 128) ? 256 : 128;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int kb = (K + BK - 1) / BK;
  int s = ws_bytes ? choose_split(tiles, kb, gfs_host::sm_count(), static_cast<size_t>(M) * N, ws_bytes) : 1;
  return s > 1 ? 2 : 1;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Split-K GEMM for callers that cannot allocate device memory (see gfs_no_alloc.h).
// The fp32 partial tiles live in this file-scope device array instead of a caller
// workspace. In host code `g_static_splitk_scratch` is only a handle for the runtime's
// symbol lookup, never a device pointer: the address the kernels get comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
// ---------------------------------------------------------------------------
#include "gfs_no_alloc.h"

static __device__ __align__(256) unsigned char g_static_splitk_scratch[GFS_NO_ALLOC_SCRATCH_BYTES];

namespace {

float* static_scratch_for_current_device() {
  static float* per_dev[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (per_dev[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_splitk_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[gfs] gfs_gemm_bf16_splitk_static: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return nullptr;
    }
    per_dev[dev] = static_cast<float*>(p);
  }
  return per_dev[dev];
}

}  // namespace

extern "C" int gfs_gemm_bf16_splitk_static(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                                           int lda, int ldb, int ldc, int ldr, int a_mn_major, int b_mn_major,
                                           int add, int splits, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || splits < 2) return GFS_NO_ALLOC_ERR_BAD_ARGUMENT;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || (add && (ldr & 7))) return GFS_NO_ALLOC_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       (add ? reinterpret_cast<uintptr_t>(R) : 0)) & 15)
    return GFS_NO_ALLOC_ERR_ALIGNMENT;
  const int kblocks = (K + BK - 1) / BK;
  if (splits > kblocks) return GFS_NO_ALLOC_ERR_BAD_ARGUMENT;
  const size_t need = static_cast<size_t>(splits) * static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(float);
  if (need > GFS_NO_ALLOC_SCRATCH_BYTES) {
    fprintf(stderr,
            "[gfs] gfs_gemm_bf16_splitk_static: %d splits of a %d x %d output need %zu bytes of partial tiles, the "
            "built-in scratch holds %u\n",
            splits, M, N, need, static_cast<unsigned>(GFS_NO_ALLOC_SCRATCH_BYTES));
    return GFS_NO_ALLOC_ERR_TOO_LARGE;
  }
  float* scratch = static_scratch_for_current_device();
  if (scratch == nullptr) return GFS_NO_ALLOC_ERR_SETUP;

  const int BN = (N > 128) ? 256 : 128;
  // tensor maps on the stack: nothing is cached or heap-allocated on this path
  CUtensorMap ta, tb;
  {
    const uint64_t a_rows = a_mn_major ? K : M, a_cols = a_mn_major ? M : K;
    const uint64_t b_rows = b_mn_major ? K : N, b_cols = b_mn_major ? N : K;
    uint64_t dims[2] = {a_cols, a_rows};
    uint64_t strides[2] = {2, static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, a_mn_major ? 64u : static_cast<uint32_t>(BM)};
    if (gfs_host::encode_tmap_bf16(&ta, A, 2, dims, strides, box) != 0) return GFS_NO_ALLOC_ERR_TENSOR_MAP;
    uint64_t dims_b[2] = {b_cols, b_rows};
    uint64_t strides_b[2] = {2, static_cast<uint64_t>(ldb) * 2};
    uint32_t box_b[2] = {64, b_mn_major ? 64u : static_cast<uint32_t>(BN)};
    if (gfs_host::encode_tmap_bf16(&tb, B, 2, dims_b, strides_b, box_b) != 0) return GFS_NO_ALLOC_ERR_TENSOR_MAP;
  }

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.ws = scratch;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.kblocks_total = kblocks;
  p.status = nullptr;  // no status buffer on this path
  p.kblocks_per_split = (kblocks + splits - 1) / splits;
  const int split = (kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split;  // no empty splits
  p.split_k = split;
  p.epi_mode = split > 1 ? EPI_PARTIAL_F32 : (add ? EPI_ADD : EPI_STORE);
  const int sms = gfs_host::sm_count();
  const int grid = std::min(p.tiles_m * p.tiles_n * split, sms);

  int rc;
  if (BN == 256) {
    if (!a_mn_major && !b_mn_major) rc = launch_variant<false, false, 256, 4>(&ta, &tb, p, grid, stream);
    else if (!a_mn_major && b_mn_major) rc = launch_variant<false, true, 256, 4>(&ta, &tb, p, grid, stream);
    else if (a_mn_major && b_mn_major) rc = launch_variant<true, true, 256, 4>(&ta, &tb, p, grid, stream);
    else rc = launch_variant<true, false, 256, 4>(&ta, &tb, p, grid, stream);
  } else {
    if (!a_mn_major && !b_mn_major) rc = launch_variant<false, false, 128, 6>(&ta, &tb, p, grid, stream);
    else if (!a_mn_major && b_mn_major) rc = launch_variant<false, true, 128, 6>(&ta, &tb, p, grid, stream);
    else if (a_mn_major && b_mn_major) rc = launch_variant<true, true, 128, 6>(&ta, &tb, p, grid, stream);
    else rc = launch_variant<true, false, 128, 6>(&ta, &tb, p, grid, stream);
  }
  if (rc != 0) return GFS_NO_ALLOC_ERR_LAUNCH;
  if (split > 1) {
    const size_t groups = static_cast<size_t>(M) * (N >> 3);
    const int threads = 256;
    const int blocks =
        static_cast<int>(std::min<size_t>((groups + threads - 1) / threads, static_cast<size_t>(sms) * 8));
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(scratch, p.C, p.R, M, N, ldc, ldr, split, add);
    if (cudaGetLastError() != cudaSuccess) return GFS_NO_ALLOC_ERR_LAUNCH;
  }
  return 0;
}
