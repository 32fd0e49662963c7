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
// Same operand layouts, addend and rotary epilogues as gemm.cu; no split-K. The fused
// collectives of gemm.cu exist here too (template parameter COMM, two extra warps per CTA):
// all-gather of A's row shards before the product (each CTA pushes a slice of the local shard
// to every peer; the producers wait per row chunk for its arrival) and reduce-scatter of the
// product's rows after it (the epilogue stores partial tiles into the owner's staging area,
// the extra warps sum what the peers delivered). Peer traffic is plain loads/stores.
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
constexpr int COMM_THREADS = 64;
constexpr int MAX_PEERS = 8;
enum CommMode : int { COMM_NONE = 0, COMM_ALLGATHER = 1, COMM_REDUCE_SCATTER = 2 };

struct CommParams {
  int world, rank;
  int rows_per_rank;                    // rows of the sharded dimension per rank (multiple of 256)
  const __nv_bfloat16* ag_src;          // all-gather: local shard [rows_per_rank, ag_cols], pitch ag_ld
  int ag_ld, ag_cols;
  __nv_bfloat16* peer_buf[MAX_PEERS];   // AG: gathered [world*rows_per_rank, ag_cols]; RS: staging [world][rows_per_rank][N]
  __nv_bfloat16* rs_out;                // reduce-scatter: out[rows_per_rank, N] = sum of partial rows (+ residual)
  const __nv_bfloat16* rs_res;
  int rs_ld_out, rs_ld_res;
  __nv_bfloat16* mc_buf;                // all-gather: multicast address of the gathered buffers, or null
  uint32_t* peer_flags[MAX_PEERS];      // flags[p][src]: progress of rank src's writes into rank p
  uint32_t target;                      // value flags[rank][src] must reach in this call
  unsigned long long wait_ns;
};
constexpr int A_BYTES = BM * BK * 2;     // 16 KB
constexpr int B_BYTES = BNH * BK * 2;    // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 8 * 4096;     // one [32 rows x 128 B] transpose buffer per epilogue warp
// Epilogue warps per CTA: 8 in the plain kernel (two per TMEM lane quarter, each taking half of the
// tile's columns, so epilogues with real work per element still hide behind the next tile's
// MMAs), also in the all-gather variant (its two push warps are cheap: 384 threads at up to 170
// registers), also in the reduce-scatter variant (with four, its epilogue - 9000 cycles per tile -
// was the longest phase of the small reduce-scatter GEMMs).
__host__ __device__ constexpr int epi_warps(int comm) { return 8 + 0 * comm; }
__host__ __device__ constexpr int threads2(int comm) { return 64 + 32 * epi_warps(comm) + (comm != 0 ? 64 : 0); }
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
  // SwiGLU fusion (template parameter SWI). 1 (forward, B = [gate rows | up rows] of a [2I, K]
  // weight): a tile pairs 128 gate columns (leader CTA's B rows) with the matching 128 up columns
  // (the other CTA's); the epilogue writes both halves of the projection (C, pitch ldc) and
  // act = silu(gate) * up (swi_act, pitch swi_ld). 2 (backward, the product is d_act [M, I]):
  // the epilogue reads gate/up from swi_gu (pitch swi_ld) and writes d_gate | d_up into C
  // ([M, 2I], pitch ldc) instead of d_act.
  int swi_I, swi_ld;
  __nv_bfloat16* swi_act;
  const __nv_bfloat16* swi_gu;
  // SWI == 3 (LM head): besides storing the logits, every epilogue warp writes the online-softmax
  // statistics (max, sum exp(x - max)) of its 128 columns of each row, computed from the
  // bf16-rounded logits: ce_partials[(tile_n * 2 + column half) * M + row]. A small kernel
  // combines them, so the cross entropy needs no pass over the logits in the forward.
  float2* ce_partials;
  // Debugging aid (gfs_gemm2_set_trace): when set, every CTA records SM-clock stamps of its phases
  // in trace[blockIdx.x * 16 + slot] (see TRACE_* below); null in normal operation.
  unsigned long long* trace;
  CommParams comm;
};

enum TraceSlot : int {
  TRACE_GLOBAL_NS = 0,   // globaltimer at kernel entry (to line CTAs up against each other)
  TRACE_ENTRY = 1,       // clock64 at kernel entry; the slots below are clock64 too
  TRACE_SETUP_DONE = 2,  // barriers initialised, TMEM allocated, cluster synchronised
  TRACE_FIRST_TMA = 3,   // producer issued its first load (after the all-gather flag wait, if any)
  TRACE_FIRST_MMA = 4,   // MMA warp committed its first tile
  TRACE_EPI_BEGIN = 5,   // first epilogue warp: first accumulator ready
  TRACE_EPI_FIRST = 6,   //   ... first tile written
  TRACE_EPI_LAST = 7,    //   ... last tile written
  TRACE_RED_BEGIN = 8,   // reduce-scatter: every source's partials have arrived
  TRACE_RED_END = 9,     //   ... this warp's share of the reduction is done
  TRACE_PUSH_DONE = 10,  // all-gather: this warp's share of the push is done
  TRACE_EXIT = 11,       // after the final cluster synchronisation
  TRACE_TILES = 12,      // tiles this CTA pair processed
};
__device__ __forceinline__ void trace_stamp(const Params2& p, int slot) {
  if (p.trace != nullptr) p.trace[blockIdx.x * 16 + slot] = static_cast<unsigned long long>(clock64());
}

__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// Tile t -> first row of the pair tile, first column, and (fused collectives) the row chunk.
// The collectives walk the ranks' row chunks in a rotated order: all-gather starts with the
// local chunk (already in place), reduce-scatter ends with it.
template <int COMM>
__device__ __forceinline__ void decode_tile2(const Params2& p, int t, int& m0, int& n0, int& chunk) {
  if (COMM == COMM_NONE) {
    m0 = (t / p.tiles_n) * 256;
    n0 = (t % p.tiles_n) * BN;
    chunk = 0;
  } else {
    const int tiles_per_chunk = (p.comm.rows_per_rank / 256) * p.tiles_n;
    const int ci = t / tiles_per_chunk;
    const int rem = t - ci * tiles_per_chunk;
    chunk = (p.comm.rank + ci + (COMM == COMM_REDUCE_SCATTER ? 1 : 0)) % p.comm.world;
    m0 = chunk * p.comm.rows_per_rank + (rem / p.tiles_n) * 256;
    n0 = (rem % p.tiles_n) * BN;
  }
}

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
// Called by all 32 lanes of the issuing warp (converged); one elected lane issues (see
// umma_ss_e in common.cuh for why the issuing loop runs on the whole warp).
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once) on the barrier at `cluster_addr` when all MMAs issued so far by the elected lane
// are done; called by all 32 lanes of the issuing warp
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(cluster_addr)
      : "memory");
}

template <bool A_MN, bool B_MN, int COMM, int SWI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads2(COMM), 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
             const __grid_constant__ CUtensorMap tmap_a_local, const Params2 p) {
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
  uint32_t* rs_sent = tmem_slot + 2;   // [MAX_PEERS] reduce-scatter: (warp, tile) units stored for each peer

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);

  if (threadIdx.x < MAX_PEERS) rs_sent[threadIdx.x] = 0u;
  if (threadIdx.x == 0) {
    if (p.trace != nullptr) p.trace[blockIdx.x * 16 + TRACE_GLOBAL_NS] = globaltimer_ns();
    trace_stamp(p, TRACE_ENTRY);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * epi_warps(COMM));
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (COMM == COMM_ALLGATHER) tma_prefetch_desc(&tmap_a_local);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs initialised, TMEM allocated
  tc_fence_after();
  // everything above ran while the preceding kernel of the stream may still have been draining
  pdl_wait();
  pdl_trigger();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  const int num_pairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;
  const int total_tiles = p.tiles_m * p.tiles_n;
  if (threadIdx.x == 0) {
    trace_stamp(p, TRACE_SETUP_DONE);
    if (p.trace != nullptr)
      p.trace[blockIdx.x * 16 + TRACE_TILES] = (total_tiles - pair + num_pairs - 1) / num_pairs;
  }

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t chunk_ready = 0;  // all-gather: chunks whose arrival has been observed
      for (int t = pair; t < total_tiles; t += num_pairs) {
        int m0, n0, chunk;
        decode_tile2<COMM>(p, t, m0, n0, chunk);
        m0 += static_cast<int>(rank) * BM;
        n0 += static_cast<int>(rank) * BNH;
        // all-gather: this rank's own chunk is read straight from its shard (tmap_a_local), so the
        // first tiles start at once; only the peers' chunks wait for their arrival in the gathered buffer
        const bool local_chunk = (COMM == COMM_ALLGATHER) && chunk == p.comm.rank;
        if (COMM == COMM_ALLGATHER && !local_chunk && !((chunk_ready >> chunk) & 1u)) {
          // rows of this chunk are written into our gathered buffer by rank `chunk`
          if (!*abort_flag &&
              !wait_flag_reached(p.comm.peer_flags[p.comm.rank] + chunk, p.comm.target, p.comm.wait_ns, p.status,
                                 0xA7000000u | (chunk << 8) | p.comm.rank))
            *abort_flag = 1u;
          fence_proxy_async_global();  // peer's generic-proxy stores -> our TMA (async proxy) loads
          chunk_ready |= 1u << chunk;
        }
        if (t == pair) trace_stamp(p, TRACE_FIRST_TMA);
        for (int kb = 0; kb < p.kblocks; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BK;
          if (!A_MN) {
            if (local_chunk) tma_load_2d_pair(sa, &tmap_a_local, bar, k0, m0 - chunk * p.comm.rows_per_rank);
            else tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tmap_a, bar, m0 + 64 * i, k0);
          }
          if (SWI == 1) {
            // n0 counts interleaved tile columns: gate rows [g0, g0 + 128) for the leader, the
            // matching up rows [I + g0, ...) for the other CTA
            const int g0 = (n0 - static_cast<int>(rank) * BNH) >> 1;
            tma_load_2d_pair(sb, &tmap_b, bar, k0, (rank == 0 ? 0 : p.swi_I) + g0);
          } else if (!B_MN) {
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
    if (leader) {  // whole warp, converged: the MMA / commit helpers elect the issuing lane
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
        if (t == pair && lane == 0) trace_stamp(p, TRACE_FIRST_MMA);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 2 + epi_warps(COMM)) {
    // ------------------------------ epilogue (both CTAs, own accumulator half) ------------------------------
    constexpr int EW = epi_warps(COMM);
    // all-gather variant: until the first accumulator is ready these warps help the two push warps
    if (COMM == COMM_ALLGATHER) {
      ag_push_rows(p.comm, static_cast<int>(threadIdx.x) - 64, COMM_THREADS + 32 * EW, 1);
      if (warp == 2 && lane == 0) trace_stamp(p, TRACE_PUSH_DONE);
    }
    bool rs_handed_over = false;                          // reduce-scatter: remote tiles handed to the signalling warp
    const int q = warp & 3;                               // TMEM lane quarter this warp may access
    const int c_begin = (EW == 8) ? ((warp - 2) >> 2) * (BN / 2) : 0;   // this warp's column range of the tile
    const int c_end = (EW == 8) ? c_begin + BN / 2 : BN;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint8_t* ebuf = epi_smem + (warp - 2) * 4096;
    const int rrow = lane >> 3;
    const int rch = lane & 7;
    const bool has_add = (p.R != nullptr);
    // The addend of a 64-column chunk is fetched one chunk ahead (across tile boundaries too), so
    // its global-memory latency is covered by the previous chunk's work instead of stalling this one.
    uint4 pre[8];
    auto load_addend = [&](uint4 (&dst)[8], int mm0, int col0) {
      const int gc = col0 + rch * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int grow = mm0 + q * 32 + i * 4 + rrow;
        dst[i] = make_uint4(0, 0, 0, 0);
        if (grow < p.M && gc + 8 <= p.N)
          dst[i] = *reinterpret_cast<const uint4*>(p.R + static_cast<size_t>(grow) * p.ldr + gc);
      }
    };
    if (has_add && pair < total_tiles) {
      int fm0, fn0, fchunk;
      decode_tile2<COMM>(p, pair, fm0, fn0, fchunk);
      load_addend(pre, fm0 + static_cast<int>(rank) * BM, fn0 + c_begin);
    }
    for (int t = pair; t < total_tiles; t += num_pairs) {
      int m0, n0, chunk;
      decode_tile2<COMM>(p, t, m0, n0, chunk);
      m0 += static_cast<int>(rank) * BM;
      mbar_wait(&tmem_full[acc], acc_phase, wctx, STATUS_TIMEOUT_TMEM_FULL);
      if (t == pair && warp == 2 && lane == 0) trace_stamp(p, TRACE_EPI_BEGIN);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (SWI == 1) {
        // accumulator columns [0,128) are gate, [128,256) the matching up columns
        const int g0 = n0 >> 1;  // first gate column of the tile
        const int sc_begin = (EW == 8) ? ((warp - 2) >> 2) * 64 : 0;
        const int sc_end = (EW == 8) ? sc_begin + 64 : 128;
#pragma unroll 1
        for (int c = sc_begin; c < sc_end; c += 32) {
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
      float ce_m = -INFINITY, ce_s = 0.f;   // SWI == 3: running statistics of this lane's row
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 64) {
        const int col0 = n0 + c;
        if (col0 >= p.N) break;
        const int gcol = col0 + rch * 8;
        uint4 cur[8];
        uint4 gq[8], uq[8];
        if (SWI == 2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int grow = m0 + q * 32 + i * 4 + rrow;
            gq[i] = make_uint4(0, 0, 0, 0);
            uq[i] = make_uint4(0, 0, 0, 0);
            if (grow < p.M && gcol + 8 <= p.N) {
              const __nv_bfloat16* gp = p.swi_gu + static_cast<size_t>(grow) * p.swi_ld + gcol;
              gq[i] = *reinterpret_cast<const uint4*>(gp);
              uq[i] = *reinterpret_cast<const uint4*>(gp + p.swi_I);
            }
          }
        }
        if (has_add) {
#pragma unroll
          for (int i = 0; i < 8; ++i) cur[i] = pre[i];
          if (c + 64 < c_end && col0 + 64 < p.N) {
            load_addend(pre, m0, col0 + 64);
          } else if (t + num_pairs < total_tiles) {
            int nm0, nn0, nchunk;
            decode_tile2<COMM>(p, t + num_pairs, nm0, nn0, nchunk);
            load_addend(pre, nm0 + static_cast<int>(rank) * BM, nn0 + c_begin);
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
        if (SWI == 3) {
          // this lane still holds its own row's 64 columns: fold their bf16-rounded values (read
          // back from the words it just wrote for the transpose) into the row's running
          // (max, sum-exp). Columns past N only exist in the last tile (warp-uniform test).
          constexpr float L2E = 1.4426950408889634f;
          const int n_valid = min(64, p.N - col0);
          uint32_t pk[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 t = *reinterpret_cast<const uint4*>(myrow + ((j ^ (lane & 7)) << 4));
            pk[4 * j + 0] = t.x; pk[4 * j + 1] = t.y; pk[4 * j + 2] = t.z; pk[4 * j + 3] = t.w;
          }
          if (n_valid < 64) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const uint32_t lo = (2 * e < n_valid) ? (pk[e] & 0xffffu) : 0xff80u;          // bf16 -inf
              const uint32_t hi = (2 * e + 1 < n_valid) ? (pk[e] & 0xffff0000u) : 0xff800000u;
              pk[e] = lo | hi;
            }
          }
          float cm0 = -INFINITY, cm1 = -INFINITY;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            cm0 = fmaxf(cm0, __uint_as_float(pk[e] << 16));
            cm1 = fmaxf(cm1, __uint_as_float(pk[e] & 0xffff0000u));
          }
          const float nm = fmaxf(ce_m, fmaxf(cm0, cm1));
          const float off = (nm == -INFINITY) ? 0.f : nm * L2E;
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            a0 += fast_exp2(fmaf(__uint_as_float(pk[e] << 16), L2E, -off));
            a1 += fast_exp2(fmaf(__uint_as_float(pk[e] & 0xffff0000u), L2E, -off));
          }
          ce_s = ce_s * fast_exp2((ce_m == -INFINITY) ? -INFINITY : (ce_m - nm) * L2E) + (a0 + a1);
          ce_m = nm;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + rrow;
          const int grow = m0 + q * 32 + r;
          uint4 w = *reinterpret_cast<const uint4*>(ebuf + r * 128 + ((rch ^ (r & 7)) << 4));
          if (SWI == 2) {
            // w holds 8 values of d_act; turn them into d_gate and d_up
            if (grow < p.M && gcol + 8 <= p.N) {
              const uint32_t* dw = &w.x;
              const uint32_t* gw = &gq[i].x;
              const uint32_t* uw = &uq[i].x;
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
                const uint4 rr = cur[i];
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
      if (SWI == 3) {
        const int row = m0 + q * 32 + lane;
        const int part = (n0 / BN) * 2 + ((EW == 8) ? ((warp - 2) >> 2) : 0);
        if (row < p.M) {
          p.ce_partials[static_cast<size_t>(part) * p.M + row] = make_float2(ce_m, ce_s);
          // with four epilogue warps a warp covers all 256 columns: the tile's second slot is empty
          if (EW != 8) p.ce_partials[static_cast<size_t>(part + 1) * p.M + row] = make_float2(-INFINITY, 0.f);
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      // the accumulator buffer may be overwritten once all epilogue warps of the pair are done
      if (COMM == COMM_REDUCE_SCATTER) {
        // Signalling the owner needs a system-scope release, which costs several microseconds (it
        // waits for every store in flight). It is therefore not done per tile: tiles for the peers
        // come first in every CTA's order; when this warp moves on to the local chunk (or runs out
        // of tiles) it hands the count to the reduction warps, which signal the owners (one release
        // per destination for the whole CTA) while the epilogue warps work on the local chunk. Local tiles only
        // need device scope.
        if (chunk != p.comm.rank) {
          if (lane == 0) atomicAdd(&rs_sent[chunk], 1u);
        } else {
          if (!rs_handed_over) {
            named_barrier_arrive(2, 32 * EW + COMM_THREADS);
            rs_handed_over = true;
          }
          if (lane == 0) red_release_gpu_add_u32(p.comm.peer_flags[chunk] + p.comm.rank, 1u);
        }
      }
      if (lane == 0) {
        mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
        if (warp == 2) {
          if (t == pair) trace_stamp(p, TRACE_EPI_FIRST);
          trace_stamp(p, TRACE_EPI_LAST);
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (COMM == COMM_REDUCE_SCATTER) {
      if (!rs_handed_over) named_barrier_arrive(2, 32 * EW + COMM_THREADS);   // CTAs without local tiles
      // tiles done: join the reduction of this rank's row chunk (second share of the vectors)
      const CommParams& c = p.comm;
      bool ok = true;
      for (int src = 0; src < c.world; ++src)
        ok = wait_flag_reached(c.peer_flags[c.rank] + src, c.target, c.wait_ns, p.status,
                               0xB8000000u | (src << 8) | c.rank) && ok;
      if (!ok) *abort_flag = 1u;
      constexpr int RED_THREADS = COMM_THREADS + 32 * EW;
      rs_reduce_rows(c.peer_buf[c.rank], c.world, c.rows_per_rank, p.N, c.rs_res, c.rs_ld_res, c.rs_out, c.rs_ld_out,
                     static_cast<size_t>(blockIdx.x) * RED_THREADS + COMM_THREADS + (threadIdx.x - 64),
                     static_cast<size_t>(gridDim.x) * RED_THREADS);
    }
  } else if (COMM == COMM_ALLGATHER) {
    // ------------------------------ all-gather push (warps 6-7) ------------------------------
    // Every CTA pushes its slice of the local shard into every rank's gathered buffer
    // (own rank first), then bumps that rank's counter for this source.
    // (the epilogue warps push too, before their first tile: see the top of the epilogue branch)
    ag_push_rows(p.comm, static_cast<int>(threadIdx.x) - (threads2(COMM) - COMM_THREADS) + 32 * epi_warps(COMM),
                 COMM_THREADS + 32 * epi_warps(COMM), 1);
  } else if (COMM == COMM_REDUCE_SCATTER) {
    // ------------------------------ reduce (warps 6-7) ------------------------------
    // Wait until every rank (this one included) has delivered all partial tiles of our row
    // chunk, then sum the staged partials in rank order, add the residual, round once.
    const CommParams& c = p.comm;
    const int ct = threadIdx.x - (threads2(COMM) - COMM_THREADS);
    // every epilogue warp of this CTA has stored its tiles for the peers: the owners learn how many (warp, tile) units this CTA delivered to each of them
    named_barrier_sync(2, 32 * epi_warps(COMM) + COMM_THREADS);
    if (ct < c.world && ct != c.rank) {
      const uint32_t n = rs_sent[ct];
      if (n != 0u) red_release_sys_add_u32(c.peer_flags[ct] + c.rank, n);   // release: cumulative over the barrier
    }
    bool ok = true;
    for (int src = 0; src < c.world; ++src)
      ok = wait_flag_reached(c.peer_flags[c.rank] + src, c.target, c.wait_ns, p.status,
                             0xB7000000u | (src << 8) | c.rank) && ok;
    if (!ok) *abort_flag = 1u;
    if (ct == 0) trace_stamp(p, TRACE_RED_BEGIN);
    // these 64 threads take the first share of the vectors; the epilogue warps take the rest once
    // their tiles are done (see the end of the epilogue loop)
    constexpr int RED_THREADS = COMM_THREADS + 32 * epi_warps(COMM);
    rs_reduce_rows(c.peer_buf[c.rank], c.world, c.rows_per_rank, p.N, c.rs_res, c.rs_ld_res, c.rs_out, c.rs_ld_out,
                   static_cast<size_t>(blockIdx.x) * RED_THREADS + ct, static_cast<size_t>(gridDim.x) * RED_THREADS);
    if (ct == 0) trace_stamp(p, TRACE_RED_END);
  }

  // nobody leaves while the partner may still touch this CTA's shared memory / barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (threadIdx.x == 0) trace_stamp(p, TRACE_EXIT);
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// Grouped weight-gradient GEMM: up to MAX_GROUP independent problems C_g[M_g, N_g] (+)= A_g^T B_g
// (A_g = [K, M_g], B_g = [K, N_g], both row-major, i.e. MN-major operands) in ONE launch. The
// weight gradients of a transformer layer are many-K, few-tile problems (hidden x hidden
// outputs, K = tokens); one by one they fill a fraction of the SMs, together they fill a wave.
// ---------------------------------------------------------------------------
constexpr int MAX_GROUP = 4;

struct GroupMaps {
  CUtensorMap a[MAX_GROUP];
  CUtensorMap b[MAX_GROUP];
};

struct GroupProblem {
  int M, N, ldc;
  int tiles_n, tile_begin, kblocks;
  int accumulate;        // add the product to C instead of overwriting it
  __nv_bfloat16* C;
};

struct GroupParams {
  int ngroups, total_tiles;
  GroupProblem g[MAX_GROUP];
  uint32_t* status;
};

__device__ __forceinline__ int group_of_tile(const GroupParams& p, int t) {
  int gi = 0;
#pragma unroll
  for (int i = 1; i < MAX_GROUP; ++i)
    if (i < p.ngroups && t >= p.g[i].tile_begin) gi = i;
  return gi;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm2_grouped_kernel(const __grid_constant__ GroupMaps maps, const __grid_constant__ GroupParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
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
    for (int i = 0; i < p.ngroups; ++i) {
      tma_prefetch_desc(&maps.a[i]);
      tma_prefetch_desc(&maps.b[i]);
    }
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  pdl_wait();
  pdl_trigger();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  const int num_pairs = gridDim.x >> 1;
  const int pair = blockIdx.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < p.total_tiles; t += num_pairs) {
        const int gi = group_of_tile(p, t);
        const GroupProblem& g = p.g[gi];
        const int lt = t - g.tile_begin;
        const int m0 = (lt / g.tiles_n) * 256 + static_cast<int>(rank) * BM;
        const int n0 = (lt % g.tiles_n) * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < g.kblocks; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BK;
#pragma unroll
          for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * 8192, &maps.a[gi], bar, m0 + 64 * i, k0);
#pragma unroll
          for (int i = 0; i < BNH / 64; ++i) tma_load_2d_pair(sb + i * 8192, &maps.b[gi], bar, n0 + 64 * i, k0);
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
    if (leader) {  // whole warp, converged: the MMA / commit helpers elect the issuing lane
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = pair; t < p.total_tiles; t += num_pairs) {
        const int kblocks = p.g[group_of_tile(p, t)].kblocks;
        mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, wctx, STATUS_TIMEOUT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(&full_bar[stage], phase, wctx, STATUS_TIMEOUT_PIPE_FULL);
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = umma_desc_sw128(sa + k * 2048, 8192, 1024);
            const uint64_t bdesc = umma_desc_sw128(sb + k * 2048, 8192, 1024);
            umma_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
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
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint8_t* ebuf = epi_smem + (warp - 2) * 4096;
    const int rrow = lane >> 3;
    const int rch = lane & 7;
    for (int t = pair; t < p.total_tiles; t += num_pairs) {
      const GroupProblem& g = p.g[group_of_tile(p, t)];
      const int lt = t - g.tile_begin;
      const int m0 = (lt / g.tiles_n) * 256 + static_cast<int>(rank) * BM;
      const int n0 = (lt % g.tiles_n) * BN;
      mbar_wait(&tmem_full[acc], acc_phase, wctx, STATUS_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 64) {
        const int col0 = n0 + c;
        if (col0 >= g.N) break;
        const int gcol = col0 + rch * 8;
        uint4 pre[8];
        if (g.accumulate) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int grow = m0 + q * 32 + i * 4 + rrow;
            pre[i] = make_uint4(0, 0, 0, 0);
            if (grow < g.M && gcol + 8 <= g.N)
              pre[i] = *reinterpret_cast<const uint4*>(g.C + static_cast<size_t>(grow) * g.ldc + gcol);
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
          if (grow < g.M && gcol + 8 <= g.N) {
            if (g.accumulate) {
              const uint4 rr = pre[i];
              const float2 x0 = unpack_bf16x2(w.x), x1 = unpack_bf16x2(w.y), x2 = unpack_bf16x2(w.z),
                           x3 = unpack_bf16x2(w.w);
              const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y), r2 = unpack_bf16x2(rr.z),
                           r3 = unpack_bf16x2(rr.w);
              w.x = pack_bf16x2(x0.x + r0.x, x0.y + r0.y);
              w.y = pack_bf16x2(x1.x + r1.x, x1.y + r1.y);
              w.z = pack_bf16x2(x2.x + r2.x, x2.y + r2.y);
              w.w = pack_bf16x2(x3.x + r3.x, x3.y + r3.y);
            }
            *reinterpret_cast<uint4*>(g.C + static_cast<size_t>(grow) * g.ldc + gcol) = w;
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// Debugging aid: device buffer of 16 uint64 per CTA that the next gemm2_kernel launches fill with
// their phase stamps (TraceSlot); null (the default) switches tracing off.
static unsigned long long* g_trace = nullptr;

template <bool A_MN, bool B_MN, int COMM = COMM_NONE, int SWI = 0>
int launch2(const CUtensorMap* ta, const CUtensorMap* tb, const Params2& p, int grid, cudaStream_t stream,
            const CUtensorMap* ta_local = nullptr) {
  auto kern = gemm2_kernel<A_MN, B_MN, COMM, SWI>;
  static bool attr_set = false;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set || attr_dev != dev) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) != cudaSuccess)
      return -10;
    attr_set = true;
    attr_dev = dev;
  }
  Params2 pt = p;
  pt.trace = g_trace;
  if (gfs_host::launch_pdl(kern, dim3(grid), dim3(threads2(COMM)), SMEM_TOTAL, stream, *ta, *tb,
                           ta_local ? *ta_local : *ta, pt) != cudaSuccess)
    return -11;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace

extern "C" {

// Debugging aid: subsequent gemm2_kernel launches (all variants, fused collectives included) write
// their per-CTA phase stamps into `buffer` (device memory, 16 uint64 per CTA of the largest grid;
// slots as in TraceSlot, SM clock cycles). Pass null to switch it off again.
void gfs_gemm2_set_trace(void* buffer) { g_trace = static_cast<unsigned long long*>(buffer); }

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

// LM head with cross-entropy statistics: C[M, N] = A[M, K] @ B[N, K]^T (both K-major) and, per row,
// the (max, sum exp(x - max)) of every 128-column slice of the bf16-rounded logits:
// partials is float2 [gfs_gemm2_ce_parts(N)][M]. Returns -20 if the problem is too small for CTA
// pairs (nothing launched).
int gfs_gemm2_ce_parts(int N) { return 2 * ((N + BN - 1) / BN); }

int gfs_gemm2_bf16_ce(const void* A, const void* B, void* C, void* partials, int M, int N, int K, int lda, int ldb,
                      int ldc, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(partials)) & 15)
    return -2;
  if (K < 256) return -20;
  const CUtensorMap* ta = gfs_host::tmap_2d_cached(A, M, K, lda, BM, 64);
  const CUtensorMap* tb = gfs_host::tmap_2d_cached(B, N, K, ldb, BNH, 64);
  if (ta == nullptr || tb == nullptr) return -3;
  Params2 p{};
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (N + BN - 1) / BN;
  p.kblocks = (K + BK - 1) / BK;
  p.status = gfs_host::status_words();
  p.rope_b = 1;
  p.ce_partials = static_cast<float2*>(partials);
  const int pairs = std::min(p.tiles_m * p.tiles_n, gfs_host::sm_count() / 2);
  return launch2<false, false, COMM_NONE, 3>(ta, tb, p, 2 * pairs, stream);
}

// SwiGLU-fused products of the MLP on CTA pairs; same contract as gfs_gemm_bf16_swiglu (gemm.cu):
//   mode 1: gu[M, 2I] = x[M, K] @ w_gu[2I, K]^T and act[M, I] = silu(gu[:, :I]) * gu[:, I:]
//           (a = x, b = w_gu, c = gu with pitch ldc, extra = act with pitch ld_extra)
//   mode 2: d_gu[M, 2I] = swiglu_backward(d_act = dy[M, K] @ w_down[K, I], gu)
//           (a = dy, b = w_down stored [K, I], c = d_gu with pitch ldc, extra = gu with pitch ld_extra)
int gfs_gemm2_bf16_swiglu(int mode, const void* a, const void* b, void* c, void* extra, int M, int I, int K, int lda,
                          int ldb, int ldc, int ld_extra, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (mode != 1 && mode != 2) return -1;
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if ((I & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7) || (ld_extra & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
       reinterpret_cast<uintptr_t>(extra)) & 15)
    return -2;
  Params2 p{};
  p.M = M; p.K = K;
  p.N = (mode == 1) ? 2 * I : I;
  p.C = static_cast<__nv_bfloat16*>(c);
  p.ldc = ldc;
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (mode == 1) ? (I + BN / 2 - 1) / (BN / 2) : (I + BN - 1) / BN;
  p.kblocks = (K + BK - 1) / BK;
  p.status = gfs_host::status_words();
  p.rope_b = 1;
  p.swi_I = I;
  p.swi_ld = ld_extra;
  if (mode == 1) p.swi_act = static_cast<__nv_bfloat16*>(extra);
  else p.swi_gu = static_cast<const __nv_bfloat16*>(extra);
  const CUtensorMap* ta = gfs_host::tmap_2d_cached(a, M, K, lda, BM, 64);
  const CUtensorMap* tb = (mode == 1) ? gfs_host::tmap_2d_cached(b, 2 * I, K, ldb, BNH, 64)
                                      : gfs_host::tmap_2d_cached(b, K, I, ldb, 64, 64);
  if (ta == nullptr || tb == nullptr) return -3;
  const int pairs = std::min(p.tiles_m * p.tiles_n, gfs_host::sm_count() / 2);
  return (mode == 1) ? launch2<false, false, COMM_NONE, 1>(ta, tb, p, 2 * pairs, stream)
                     : launch2<false, true, COMM_NONE, 2>(ta, tb, p, 2 * pairs, stream);
}

// Fused collective + GEMM on CTA pairs; same contract as gfs_gemm_bf16_comm (gemm.cu) with the
// extra requirement that M/world is a multiple of 256. Returns -20 when the problem does not
// qualify, in which case the caller uses the single-CTA kernel (nothing has been launched and
// *target_inout is unchanged).
static int gemm2_comm_impl(int mode, const void* a, int lda, const void* B, int ldb, void* out, int ldo,
                           const void* residual, int ldr, int M, int N, int K, int b_mn_major, int world, int rank,
                           const unsigned long long* peer_bufs, const unsigned long long* peer_flags,
                           unsigned int* target_inout, const void* rope_cos, const void* rope_sin, int rope_cols,
                           int rope_d, int rope_b, long long wait_ns, void* ce_partials, void* stream_,
                           int swi_mode = 0, void* swi_extra = nullptr, int swi_ld = 0) {
  // swi_mode 1 / 2 (all-gather only): the SwiGLU epilogues of gfs_gemm2_bf16_swiglu. Mode 1: N = 2I
  // columns of the [gate | up] projection, out = gu [M, 2I], swi_extra = act [M, I]. Mode 2: N = I
  // columns of d_act, B stored [K, I], out = d_gu [M, 2I], swi_extra = gu [M, 2I].
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (mode != COMM_ALLGATHER && mode != COMM_REDUCE_SCATTER) return -1;
  if (swi_mode != 0 && (mode != COMM_ALLGATHER || ce_partials != nullptr || rope_cos != nullptr || residual ||
                        swi_extra == nullptr || (swi_ld & 7) || (reinterpret_cast<uintptr_t>(swi_extra) & 15) ||
                        b_mn_major != (swi_mode == 2) || (swi_mode == 1 && (N & 15))))
    return -1;
  if (ce_partials != nullptr && (mode != COMM_ALLGATHER || b_mn_major || rope_cos != nullptr)) return -1;
  if (world < 2 || world > MAX_PEERS || rank < 0 || rank >= world) return -1;
  if (M <= 0 || N <= 0 || K <= 0 || (M % world) != 0) return -1;
  if (((M / world) % 256) != 0 || N < 256 || K < 256) return -20;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldo & 7) || (residual && (ldr & 7))) return -1;
  const int rows_per_rank = M / world;
  Params2 p{};
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / 256;
  p.tiles_n = (N + BN - 1) / BN;
  p.kblocks = (K + BK - 1) / BK;
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
  const int pairs = std::min(p.tiles_m * p.tiles_n, gfs_host::sm_count() / 2);
  const int grid = 2 * pairs;
  const void* a_base;
  int a_ld;
  unsigned int increment;
  if (mode == COMM_ALLGATHER) {
    c.ag_src = static_cast<const __nv_bfloat16*>(a);
    c.ag_ld = lda;
    c.ag_cols = K;
    a_base = c.peer_buf[rank];   // the GEMM reads the local gathered buffer
    a_ld = K;
    p.C = static_cast<__nv_bfloat16*>(out);
    p.ldc = ldo;
    increment = static_cast<unsigned int>(grid);   // every CTA of a source signals once per destination
  } else {
    a_base = a;
    a_ld = lda;
    c.rs_out = static_cast<__nv_bfloat16*>(out);
    c.rs_ld_out = ldo;
    c.rs_res = static_cast<const __nv_bfloat16*>(residual);
    c.rs_ld_res = ldr;
    increment = static_cast<unsigned int>((rows_per_rank / 256) * p.tiles_n * 2 * epi_warps(COMM_REDUCE_SCATTER));  // (warp, tile) units per pair tile
  }
  if ((reinterpret_cast<uintptr_t>(a_base) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return -2;
  const CUtensorMap* ta = gfs_host::tmap_2d_cached(a_base, M, K, a_ld, BM, 64);
  const CUtensorMap* tb = b_mn_major ? gfs_host::tmap_2d_cached(B, K, N, ldb, 64, 64)
                                     : gfs_host::tmap_2d_cached(B, N, K, ldb, BNH, 64);
  if (ta == nullptr || tb == nullptr) return -3;
  const CUtensorMap* ta_local = nullptr;   // all-gather: this rank's own shard, read in place
  if (mode == COMM_ALLGATHER) {
    if (reinterpret_cast<uintptr_t>(a) & 15) return -2;
    ta_local = gfs_host::tmap_2d_cached(a, rows_per_rank, K, lda, BM, 64);
    if (ta_local == nullptr) return -3;
  }
  if (swi_mode == 1) {
    p.swi_I = N / 2;
    p.tiles_n = (p.swi_I + BN / 2 - 1) / (BN / 2);
    p.swi_ld = swi_ld;
    p.swi_act = static_cast<__nv_bfloat16*>(swi_extra);
  } else if (swi_mode == 2) {
    p.swi_I = N;
    p.swi_ld = swi_ld;
    p.swi_gu = static_cast<const __nv_bfloat16*>(swi_extra);
  }
  *target_inout += increment;
  c.target = *target_inout;
  if (swi_mode == 1) return launch2<false, false, COMM_ALLGATHER, 1>(ta, tb, p, grid, stream, ta_local);
  if (swi_mode == 2) return launch2<false, true, COMM_ALLGATHER, 2>(ta, tb, p, grid, stream, ta_local);
  if (ce_partials != nullptr) {
    p.ce_partials = static_cast<float2*>(ce_partials);
    return launch2<false, false, COMM_ALLGATHER, 3>(ta, tb, p, grid, stream, ta_local);
  }
  if (mode == COMM_ALLGATHER)
    return b_mn_major ? launch2<false, true, COMM_ALLGATHER>(ta, tb, p, grid, stream, ta_local)
                      : launch2<false, false, COMM_ALLGATHER>(ta, tb, p, grid, stream, ta_local);
  return b_mn_major ? launch2<false, true, COMM_REDUCE_SCATTER>(ta, tb, p, grid, stream)
                    : launch2<false, false, COMM_REDUCE_SCATTER>(ta, tb, p, grid, stream);
}

int gfs_gemm2_bf16_comm(int mode, const void* a, int lda, const void* B, int ldb, void* out, int ldo,
                        const void* residual, int ldr, int M, int N, int K, int b_mn_major, int world, int rank,
                        const unsigned long long* peer_bufs, const unsigned long long* peer_flags,
                        unsigned int* target_inout, const void* rope_cos, const void* rope_sin, int rope_cols,
                        int rope_d, int rope_b, long long wait_ns, void* stream_) {
  return gemm2_comm_impl(mode, a, lda, B, ldb, out, ldo, residual, ldr, M, N, K, b_mn_major, world, rank, peer_bufs,
                         peer_flags, target_inout, rope_cos, rope_sin, rope_cols, rope_d, rope_b, wait_ns, nullptr,
                         stream_);
}

// Tensor-parallel SwiGLU MLP under sequence parallelism: the all-gather GEMMs with the SwiGLU
// epilogues of gfs_gemm2_bf16_swiglu.
//   mode 1: a = this rank's shard of x [M/world, K], B = w_gu [2I, K];  out = gu [M, 2I] (pitch ldo),
//           extra = act [M, I] = silu(gate) * up (pitch ld_extra)
//   mode 2: a = this rank's shard of dOut [M/world, K], B = w_down stored [K, I]; out = d_gu [M, 2I],
//           extra = gu [M, 2I] (the forward's projection)
// peer_bufs[p] = rank p's gathered [M, K] buffer. Returns -20 like gfs_gemm2_bf16_comm.
int gfs_gemm2_bf16_comm_swiglu(int swi_mode, const void* a, int lda, const void* B, int ldb, void* out, int ldo,
                               void* extra, int ld_extra, int M, int I, int K, int world, int rank,
                               const unsigned long long* peer_bufs, const unsigned long long* peer_flags,
                               unsigned int* target_inout, long long wait_ns, void* stream_) {
  if (swi_mode != 1 && swi_mode != 2) return -1;
  if ((I & 7) || I < 256) return (I & 7) ? -1 : -20;
  return gemm2_comm_impl(COMM_ALLGATHER, a, lda, B, ldb, out, ldo, nullptr, 0, M, swi_mode == 1 ? 2 * I : I, K,
                         swi_mode == 2 ? 1 : 0, world, rank, peer_bufs, peer_flags, target_inout, nullptr, nullptr, 0, 0,
                         1, wait_ns, nullptr, stream_, swi_mode, extra, ld_extra);
}

// Vocabulary-parallel LM head under sequence parallelism: the all-gather GEMM
// (logits[M, N] = gather(a)[M, K] @ B[N, K]^T, B K-major) whose epilogue also writes the
// cross-entropy statistics of gfs_gemm2_bf16_ce: partials is float2 [gfs_gemm2_ce_parts(N)][M]
// (the second slot of every 256-column tile holds the empty pair (-inf, 0): four epilogue warps
// per CTA here, each covering the tile's full width). Returns -20 like gfs_gemm2_bf16_comm.
int gfs_gemm2_bf16_allgather_ce(const void* a, int lda, const void* B, int ldb, void* out, int ldo, void* partials,
                                int M, int N, int K, int world, int rank, const unsigned long long* peer_bufs,
                                const unsigned long long* peer_flags, unsigned int* target_inout, long long wait_ns,
                                void* stream_) {
  if (partials == nullptr || (reinterpret_cast<uintptr_t>(partials) & 15)) return -2;
  return gemm2_comm_impl(COMM_ALLGATHER, a, lda, B, ldb, out, ldo, nullptr, 0, M, N, K, 0, world, rank, peer_bufs,
                         peer_flags, target_inout, nullptr, nullptr, 0, 0, 1, wait_ns, partials, stream_);
}

// Grouped weight gradients: for g < n, C_g[M_g, N_g] (+)= A_g^T B_g with A_g = [K_g, M_g] (pitch lda_g),
// B_g = [K_g, N_g] (pitch ldb_g), all bf16 row-major, fp32 accumulation, one launch. n <= 4.
// accumulate_g != 0 adds the product to the existing C_g (rounded once).
int gfs_gemm2_wgrad_grouped(int n, const unsigned long long* A, const unsigned long long* B,
                            const unsigned long long* C, const int* M, const int* N, const int* K, const int* lda,
                            const int* ldb, const int* ldc, const int* accumulate, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (n <= 0) return 0;
  if (n > MAX_GROUP) return -1;
  GroupMaps maps;
  GroupParams p{};
  p.ngroups = n;
  p.status = gfs_host::status_words();
  int total = 0;
  for (int i = 0; i < n; ++i) {
    if (M[i] <= 0 || N[i] <= 0 || K[i] <= 0) return -1;
    if ((N[i] & 7) || (M[i] & 7) || (lda[i] & 7) || (ldb[i] & 7) || (ldc[i] & 7)) return -1;
    if ((A[i] | B[i] | C[i]) & 15) return -2;
    const CUtensorMap* ta = gfs_host::tmap_2d_cached(reinterpret_cast<const void*>(A[i]), K[i], M[i], lda[i], 64, 64);
    const CUtensorMap* tb = gfs_host::tmap_2d_cached(reinterpret_cast<const void*>(B[i]), K[i], N[i], ldb[i], 64, 64);
    if (ta == nullptr || tb == nullptr) return -3;
    maps.a[i] = *ta;
    maps.b[i] = *tb;
    GroupProblem& g = p.g[i];
    g.M = M[i]; g.N = N[i]; g.ldc = ldc[i];
    g.tiles_n = (N[i] + BN - 1) / BN;
    g.tile_begin = total;
    g.kblocks = (K[i] + BK - 1) / BK;
    g.accumulate = accumulate[i];
    g.C = reinterpret_cast<__nv_bfloat16*>(C[i]);
    total += ((M[i] + 255) / 256) * g.tiles_n;
  }
  for (int i = n; i < MAX_GROUP; ++i) {
    maps.a[i] = maps.a[0];
    maps.b[i] = maps.b[0];
    p.g[i] = p.g[0];
    p.g[i].tile_begin = 0x7fffffff;
  }
  p.total_tiles = total;
  static bool attr_set = false;
  static int attr_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set || attr_dev != dev) {
    if (cudaFuncSetAttribute(gemm2_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) !=
        cudaSuccess)
      return -10;
    attr_set = true;
    attr_dev = dev;
  }
  const int pairs = std::min(total, gfs_host::sm_count() / 2);
  if (gfs_host::launch_pdl(gemm2_grouped_kernel, dim3(2 * pairs), dim3(THREADS), SMEM_TOTAL, stream, maps, p) !=
      cudaSuccess)
    return -11;
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
