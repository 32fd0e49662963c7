// Causal flash attention forward and backward for sm_100a (head_dim 64 or 128, bf16).
//
// All matrix products run on tcgen05.mma with fp32 accumulators in TMEM; operands are
// staged by TMA straight out of strided tensors (for the model: the packed
// [S,B,3,nh,D] qkv buffer, so no permute/contiguous copies exist), and the output is
// written directly in [S,B,nh*D] layout.
//
// Forward (one CTA per 128 query rows of one (batch, head); 6 warps):
//   warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 softmax (one thread per query row).
//   Per 128-key block: S = Q K^T -> TMEM; softmax threads read their row with tcgen05.ld,
//   keep the running max / sum, write P (bf16) into 128B-swizzled shared memory; the MMA
//   warp then computes P V into a second TMEM tile that the softmax threads fold into
//   their register-resident output row (rescaled by exp(m_old - m_new)). S, P and PV are
//   double buffered so block j+1's QK^T overlaps block j's softmax.
//
// Backward (two kernels from one template, deterministic, no atomics):
//   mode 0: one CTA per 128 keys   -> dK, dV, streaming 64-query tiles
//   mode 1: one CTA per 128 queries -> dQ,     streaming 64-key tiles
//   Both recompute P = exp(S*scale - LSE), dS = P * (dP - D) from two score MMAs
//   (X = R1 T1^T, Y = R2 T2^T), write P / dS (bf16) to shared memory and accumulate
//   dV += P^T dO, dK += dS^T Q (mode 0) or dQ += dS K (mode 1) in TMEM. The streamed tile
//   is consumed twice from the same shared-memory bytes: K-major for the score MMA and
//   MN-major for the gradient MMA.
//
// Reference counterparts: core/myFlashAttn.py:460-728 (_attn_fwd), :740-790 (pre-pass),
// :805-1066 (_attn_bwd_LoopQ), :1079-1317 (_attn_bwd_LoopKV).
#include <cstdlib>
#include <algorithm>
#include <type_traits>

#include "common.cuh"

using namespace gfs;

namespace {

constexpr int ATT_THREADS = 192;
constexpr float LOG2E_F = 1.4426950408889634f;

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}

// A K-major [rows x K] (64-column blocks a_blk bytes apart), B K-major [N x K] (blocks b_blk apart).
// Classifies a (32-row warp slice) x (column chunk) block of the score matrix against the
// causal / sequence-end mask: 0 = every element alive, 1 = mixed, 2 = every element dead.
// KEY_ROWS: rows are key positions and columns are query positions (dead when col < row);
// otherwise rows are queries and columns are keys (dead when col > row). Warp-uniform.
// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool KEY_ROWS>
__device__ __forceinline__ int mask_class(int row_min, int row_max, int col_min, int col_max, bool causal, int S) {
  if (col_min >= S) return 2;
  bool all_alive = col_max < S, all_dead = false;
  if (causal) {
    if (KEY_ROWS) {
      all_alive = all_alive && col_min >= row_max;
      all_dead = col_max < row_min;
    } else {
      all_alive = all_alive && col_max <= row_min;
      all_dead = col_min > row_max;
    }
  }
  return all_dead ? 2 : (all_alive ? 0 : 1);
}

// The shared-memory descriptors are built once per call and advanced by adding the byte offset
// (in 16-byte units) to their start-address field: the tiles are 1024-byte aligned and the
// offsets small, so the 14-bit field never carries. The issuing thread competes with the
// compute warps for issue slots, so every instruction saved per MMA shortens the chain.
template <int KSTEPS>
__device__ __forceinline__ void mma_kk(uint32_t d, uint32_t a, uint32_t a_blk, uint32_t b, uint32_t b_blk,
                                       uint32_t idesc, bool accumulate) {
  const uint64_t ad0 = umma_desc_sw128(a, 16, 1024);
  const uint64_t bd0 = umma_desc_sw128(b, 16, 1024);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const uint64_t ad = ad0 + (((ks >> 2) * a_blk + (ks & 3) * 32) >> 4);
    const uint64_t bd = bd0 + (((ks >> 2) * b_blk + (ks & 3) * 32) >> 4);
    umma_ss_e(d, ad, bd, idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}
// A K-major; B MN-major: stored as [K rows x N] in 64-column blocks b_blk bytes apart
// (each block: K rows of 128 B).
template <int KSTEPS>
__device__ __forceinline__ void mma_kmn(uint32_t d, uint32_t a, uint32_t a_blk, uint32_t b, uint32_t b_blk,
                                        uint32_t idesc, bool accumulate) {
  const uint64_t ad0 = umma_desc_sw128(a, 16, 1024);
  const uint64_t bd0 = umma_desc_sw128(b, b_blk, 1024);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const uint64_t ad = ad0 + (((ks >> 2) * a_blk + (ks & 3) * 32) >> 4);
    const uint64_t bd = bd0 + ((ks * 2048) >> 4);
    umma_ss_e(d, ad, bd, idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// A in tensor memory (8 columns per 16-wide K step); B MN-major as in mma_kmn.
template <int KSTEPS>
__device__ __forceinline__ void mma_tmn(uint32_t d, uint32_t a_tmem, uint32_t b, uint32_t b_blk, uint32_t idesc,
                                        bool accumulate) {
  const uint64_t bd0 = umma_desc_sw128(b, b_blk, 1024);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const uint64_t bd = bd0 + ((ks * 2048) >> 4);
    umma_ts_e(d, a_tmem + ks * 8, bd, idesc, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// ---------------------------------------------------------------------------
// Epilogue stores. An accumulator row lives in one thread, so a direct store instruction writes 16
// bytes to each of 32 different rows: 32 passes through the load/store unit per instruction, which
// made the epilogues of these kernels LSU-bound (about 1,000 cycles per 128 x 64 output tile). The
// rows are therefore transposed through a per-warp staging area in shared memory (XOR-swizzled, free
// of bank conflicts both ways) and leave as whole 64- or 128-byte row segments.
// ---------------------------------------------------------------------------
// 32 rows x 32 bf16 columns; w = this lane's row (16 packed words); stage: 2 KB of this warp.
__device__ __forceinline__ void store_rows_32x32(uint8_t* stage, const uint32_t (&w)[16], int lane,
                                                 __nv_bfloat16* g0, long long row_stride, int rows_valid) {
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4)
    *reinterpret_cast<uint4*>(stage + lane * 64 + ((q4 ^ ((lane >> 1) & 3)) << 4)) =
        make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = (lane >> 2) + 8 * i;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 64 + (((lane & 3) ^ ((row >> 1) & 3)) << 4));
    if (row < rows_valid) *reinterpret_cast<uint4*>(g0 + row * row_stride + (lane & 3) * 8) = v;
  }
  __syncwarp();
}

// 32 rows x 64 bf16 columns; w = this lane's row (32 packed words); stage: 4 KB of this warp.
__device__ __forceinline__ void store_rows_32x64(uint8_t* stage, const uint32_t (&w)[32], int lane,
                                                 __nv_bfloat16* g0, long long row_stride, int rows_valid) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch)
    *reinterpret_cast<uint4*>(stage + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
        make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = (lane >> 3) + 4 * i;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 128 + (((lane & 7) ^ (row & 7)) << 4));
    if (row < rows_valid) *reinterpret_cast<uint4*>(g0 + row * row_stride + (lane & 7) * 8) = v;
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
struct FwdParams {
  __nv_bfloat16* O;
  long long o_ss, o_bs, o_hs;  // element strides: sequence, batch, head
  float* lse;                  // [B, nh, S_pad]
  int S, S_pad, B, nh;
  float scale;
  int causal;
  uint32_t* status;
};

// NBUF = 2: S / P / PV tiles double buffered, one CTA per SM (head_dim 128).
// NBUF = 1: single buffers, half the shared memory and TMEM, so two CTAs share an SM and
//           hide each other's softmax / MMA latencies (head_dim 64).
template <int D, int NBUF>
__global__ void __launch_bounds__(ATT_THREADS, NBUF == 1 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const FwdParams p) {
  constexpr int DB = D / 64;
  constexpr int TILE_BYTES = DB * 16384;  // [128 x D] bf16 as DB swizzled blocks
  constexpr int P_BYTES = 32768;          // [128 x 128] bf16 as 2 swizzled blocks
  constexpr uint32_t TMEM_COLS = (NBUF == 2) ? 512 : 256;
  constexpr uint32_t OP_COL = NBUF * 128;  // PV tiles start after the S tiles
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;  // the launcher requests exactly the bytes used; the base must be 1024-aligned
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + TILE_BYTES;
  uint8_t* Vs = Ks + 2 * TILE_BYTES;
  uint8_t* Ps = Vs + 2 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + NBUF * P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;
  uint64_t* s_empty = bars + 11;
  uint64_t* p_full = bars + 13;
  uint64_t* p_empty = bars + 15;
  uint64_t* o_full = bars + 17;
  uint64_t* o_empty = bars + 19;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (smem_u32(smem_raw) & 1023u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) record_status(p.status, STATUS_BAD_ARGUMENT, 0x5a11u);
    return;
  }
  const int qt = gridDim.x - 1 - blockIdx.x;  // heaviest (most key blocks) first
  const int bh = blockIdx.y;
  const int b = bh / p.nh;
  const int h = bh % p.nh;
  const int n_blocks_all = (p.S + 127) >> 7;
  const int n_kv = p.causal ? min(qt + 1, n_blocks_all) : n_blocks_all;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4);
      mbar_init(&p_empty[i], 1);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();       // set-up above may overlap the tail of the preceding kernel (programmatic launch)
  pdl_trigger();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_4d(Qs + db * 16384, &tq, q_full, db * 64, qt * 128, h, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1u;
        mbar_wait(&k_empty[st], par, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
        mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db)
          tma_load_4d(Ks + st * TILE_BYTES + db * 16384, &tk, &k_full[st], db * 64, j * 128, h, b);
        mbar_wait(&v_empty[st], par, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
        mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db)
          tma_load_4d(Vs + st * TILE_BYTES + db * 16384, &tv, &v_full[st], db * 64, j * 128, h, b);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    {  // whole warp, converged: the MMA / commit helpers elect the issuing lane
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      const uint32_t q_addr = smem_u32(Qs);
      mbar_wait(q_full, 0, wctx, STATUS_TIMEOUT_PIPE_FULL);
      auto issue_s = [&](int j) {
        const int st = j & 1;                       // K/V stage
        const uint32_t par = (j >> 1) & 1;
        const int sb = (NBUF == 2) ? (j & 1) : 0;   // S / P / PV buffer
        const uint32_t spar = (NBUF == 2) ? ((j >> 1) & 1) : (j & 1);
        mbar_wait(&k_full[st], par, wctx, STATUS_TIMEOUT_PIPE_FULL);
        mbar_wait(&s_empty[sb], spar ^ 1u, wctx, STATUS_TIMEOUT_SOFTMAX);
        tc_fence_after();
        mma_kk<D / 16>(tmem_base + sb * 128, q_addr, 16384, smem_u32(Ks + st * TILE_BYTES), 16384, idesc_s, false);
        umma_commit_e(&s_full[sb]);
        umma_commit_e(&k_empty[st]);
      };
      issue_s(0);
      for (int j = 0; j < n_kv; ++j) {
        if (j + 1 < n_kv) issue_s(j + 1);
        const int st = j & 1;
        const uint32_t par = (j >> 1) & 1;
        const int sb = (NBUF == 2) ? (j & 1) : 0;
        const uint32_t spar = (NBUF == 2) ? ((j >> 1) & 1) : (j & 1);
        mbar_wait(&p_full[sb], spar, wctx, STATUS_TIMEOUT_SOFTMAX);
        mbar_wait(&v_full[st], par, wctx, STATUS_TIMEOUT_PIPE_FULL);
        mbar_wait(&o_empty[sb], spar ^ 1u, wctx, STATUS_TIMEOUT_SOFTMAX);
        tc_fence_after();
        mma_kmn<8>(tmem_base + OP_COL + sb * D, smem_u32(Ps + sb * P_BYTES), 16384, smem_u32(Vs + st * TILE_BYTES),
                   16384, idesc_o, false);
        umma_commit_e(&o_full[sb]);
        umma_commit_e(&v_empty[st]);
        umma_commit_e(&p_empty[sb]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;       // row inside the query tile
    const int row_g = qt * 128 + r;          // query position
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * LOG2E_F;
    float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;

    auto fold_pv = [&](int j, float alpha) {
      const int st = (NBUF == 2) ? (j & 1) : 0;
      mbar_wait(&o_full[st], (NBUF == 2) ? ((j >> 1) & 1) : (j & 1), wctx, STATUS_TIMEOUT_SOFTMAX);
      tc_fence_after();
      const uint32_t o_addr = tmem_base + lane_base + OP_COL + st * D;
      uint32_t wa[32], wb[32];
      tmem_ld_32x32(o_addr, wa);
#pragma unroll
      for (int c = 0; c < D; c += 64) {
        tmem_ld_wait_for(wa);
        tmem_ld_32x32(o_addr + c + 32, wb);
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c + e] = fmaf(o[c + e], alpha, __uint_as_float(wa[e]));
        tmem_ld_wait_for(wb);
        if (c + 64 < D) tmem_ld_32x32(o_addr + c + 64, wa);
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c + 32 + e] = fmaf(o[c + 32 + e], alpha, __uint_as_float(wb[e]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty[st]);
    };

    for (int j = 0; j < n_kv; ++j) {
      const int st = (NBUF == 2) ? (j & 1) : 0;
      const uint32_t par = (NBUF == 2) ? ((j >> 1) & 1) : (j & 1);
      const bool need_mask = (p.causal && j == qt) || ((j + 1) * 128 > p.S);
      mbar_wait(&s_full[st], par, wctx, STATUS_TIMEOUT_SOFTMAX);
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_base + st * 128;
      // pass 1: row maximum (TMEM loads double buffered against the arithmetic)
      float mx = -INFINITY;
      uint32_t va[32], vb[32];
      // Diagonal / tail block: dead scores become -inf in the registers and the block runs the same
      // max / exponential code as every other block (a separate masked copy of that code executes
      // once per CTA from a cold instruction cache and cost more than two unmasked blocks).
      auto mask_chunk = [&](uint32_t (&v)[32], int c) {
        if (need_mask) {
          const int lim_c = p.causal ? row_g - j * 128 - c : 0x7fffffff;   // last live column of the chunk
          const int lim = min(lim_c, p.S - 1 - j * 128 - c);
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = (e > lim) ? 0xff800000u : v[e];
        }
      };
      auto max_chunk = [&](uint32_t (&v)[32], int c) {
        mask_chunk(v, c);
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v[e]));
      };
      tmem_ld_32x32(s_addr + 0, va);
      tmem_ld_wait_for(va);
      tmem_ld_32x32(s_addr + 32, vb);
      max_chunk(va, 0);
      tmem_ld_wait_for(vb);
      tmem_ld_32x32(s_addr + 64, va);
      max_chunk(vb, 32);
      tmem_ld_wait_for(va);
      tmem_ld_32x32(s_addr + 96, vb);
      max_chunk(va, 64);
      tmem_ld_wait_for(vb);
      tmem_ld_32x32(s_addr + 0, va);  // first chunk of pass 2
      max_chunk(vb, 96);
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // row with no live key so far
      const float alpha = fast_exp2((m - m_use) * sl2);
      const float moff = m_use * sl2;
      mbar_wait(&p_empty[st], par ^ 1u, wctx, STATUS_TIMEOUT_SOFTMAX);
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float rs = 0.f;
      uint8_t* prow = Ps + st * P_BYTES + r * 128;
      auto prob_chunk = [&](uint32_t (&v)[32], int c) {
        mask_chunk(v, c);
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float x0 = fast_exp2(fmaf(__uint_as_float(v[e]), sl2, -moff));
          const float x1 = fast_exp2(fmaf(__uint_as_float(v[e + 1]), sl2, -moff));
          rs += x0 + x1;
          packed[e >> 1] = pack_bf16x2(x0, x1);
        }
        uint8_t* blk = prow + (c >> 6) * 16384;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint4 w = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(blk + ((((chunk0 + q4) ^ (r & 7)) & 7) << 4)) = w;
        }
      };
      tmem_ld_wait_for(va);
      tmem_ld_32x32(s_addr + 32, vb);
      prob_chunk(va, 0);
      tmem_ld_wait_for(vb);
      tmem_ld_32x32(s_addr + 64, va);
      prob_chunk(vb, 32);
      tmem_ld_wait_for(va);
      tmem_ld_32x32(s_addr + 96, vb);
      prob_chunk(va, 64);
      tmem_ld_wait_for(vb);
      prob_chunk(vb, 96);
      l = l * alpha + rs;
      m = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[st]);
        mbar_arrive(&p_full[st]);
      }
      if (j > 0) fold_pv(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    fold_pv(n_kv - 1, alpha_prev);

    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    {
      // every P V MMA has completed (the last fold waited for it): the P buffer serves as staging
      uint8_t* stage = Ps + (r >> 5) * 4096;
      const int row0 = row_g - lane;
      __nv_bfloat16* g0 = p.O + row0 * p.o_ss + b * p.o_bs + h * p.o_hs;
#pragma unroll
      for (int hf = 0; hf < D / 64; ++hf) {
        uint32_t ow[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) ow[e] = pack_bf16x2(o[hf * 64 + 2 * e] * inv_l, o[hf * 64 + 2 * e + 1] * inv_l);
        store_rows_32x64(stage, ow, lane, g0 + hf * 64, p.o_ss, p.S - row0);
      }
    }
    if (row_g < p.S_pad) {
      const float mm = (m == -INFINITY) ? 0.f : m;
      p.lse[static_cast<size_t>(bh) * p.S_pad + row_g] = mm * p.scale + logf(fmaxf(l, 1e-37f));
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Forward, head_dim 64: two 128-row query tiles per CTA.
//
// One CTA per SM; warps 2-5 run the softmax of tile A and warps 6-9 that of tile B (one thread
// per query row, so no cross-thread reductions), which gives every scheduler two independent
// softmax warps while K/V tiles are fetched once for 256 query rows. S, P V and P each live
// in tensor memory (S_A S_B | PV_A PV_B | P_A P_B = 512 columns): the probabilities are
// handed to the P V MMA as its TMEM A operand, nothing of the softmax goes through shared
// memory. K/V use a 4-stage ring (three: 111.1 us, four: 109.4 us at the GPT-124M shape with an
// earlier version; six stages measured 1.5 % slower than four with this one).
// ---------------------------------------------------------------------------
constexpr int FWD64_THREADS = 64 + 256;
constexpr int FWD64_KS = 4;
constexpr int FWD64_SMEM = 2 * 16384 + FWD64_KS * 32768 + 512;

// Persistent: each CTA walks work items (pair of query tiles, batch*head), heaviest pairs
// first, so barrier set-up, the TMEM allocation and the CTA launch gap are paid once per SM
// instead of once per item (at sequence length 1024 they were ~45 % of the kernel's time).
// All barrier parities therefore run on counters that continue across items.
//
// The output accumulates in tensor memory (P V issued with accumulate) instead of being
// folded into registers after every key block, and the running maximum is only raised when it
// grows by more than 2^8 (any consistent offset gives the same softmax; the stale one keeps
// exp2 arguments <= 8). Raising it rescales the accumulator in tensor memory, which after the
// first blocks is rare. This frees the 64 accumulator registers per thread, so a block's 128
// scores are loaded once and stay in registers for both the maximum and the exponentials.
__global__ void __launch_bounds__(FWD64_THREADS, 1)
flash_fwd64_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const FwdParams p, int n_pairs, int n_items) {
  constexpr int D = 64;
  constexpr int KS = FWD64_KS;
  constexpr uint32_t S_COL = 0, OP_COL = 256, P_COL = 384;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* Qs = smem_raw;                    // [2][128 x 64]
  uint8_t* Ks = Qs + 2 * 16384;              // [KS][128 x 64]
  uint8_t* Vs = Ks + KS * 16384;             // [KS][128 x 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + KS * 16384);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;               // [KS]
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + KS;
  uint64_t* s_full = v_empty + KS;           // [2] per query tile
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint64_t* o_empty = o_full + 2;
  uint64_t* s_free = o_empty + 2;            // [2] the tile's scores have been read out of tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) record_status(p.status, STATUS_BAD_ARGUMENT, 0x5a12u);
    return;
  }
  const int nb = (p.S + 127) >> 7;
  const int BH = p.B * p.nh;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < KS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_empty[i], 4);
      mbar_init(&s_free[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();       // set-up above may overlap the tail of the preceding kernel (programmatic launch)
  pdl_trigger();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  // Work items are dealt to the CTAs in a snake (left to right, then right to left), which
  // evens out the per-CTA totals of the descending item weights; an item past the end can
  // only occur in a CTA's last round.
  const int G = static_cast<int>(gridDim.x);
  auto snake = [&](int rnd) {
    return rnd * G + ((rnd & 1) ? G - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x));
  };
  // decode of work item w: pairs in descending order (most key blocks first), then batch*head
  auto decode = [&](int w, int& qp, int& bh, int& na, int& nbk) {
    qp = n_pairs - 1 - w / BH;
    bh = w % BH;
    const int qa = 2 * qp, qb = 2 * qp + 1;
    na = p.causal ? min(qa + 1, nb) : nb;
    nbk = (qb < nb) ? (p.causal ? min(qb + 1, nb) : nb) : 0;
  };

  if (warp == 0) {
    if (lane == 0) {
      int g = 0;      // key blocks loaded so far (ring position)
      for (int rnd = 0; rnd * G < n_items; ++rnd) {
        const int w = snake(rnd);
        if (w >= n_items) break;
        const int item = rnd;
        int qp, bh, na, nbk;
        decode(w, qp, bh, na, nbk);
        const int b = bh / p.nh, h = bh % p.nh;
        const int n_kv = max(na, nbk);
        mbar_wait(q_empty, (item & 1) ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);  // previous item's S MMAs done
        mbar_arrive_expect_tx(q_full, 2 * 16384);
        tma_load_4d(Qs, &tq, q_full, 0, (2 * qp) * 128, h, b);
        tma_load_4d(Qs + 16384, &tq, q_full, 0, (2 * qp + 1) * 128, h, b);   // rows past S are zero-filled
        for (int j = 0; j < n_kv; ++j, ++g) {
          const int st = g % KS;
          const uint32_t par = ((g / KS) & 1) ^ 1u;
          mbar_wait(&k_empty[st], par, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
          mbar_arrive_expect_tx(&k_full[st], 16384);
          tma_load_4d(Ks + st * 16384, &tk, &k_full[st], 0, j * 128, h, b);
          mbar_wait(&v_empty[st], par, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
          mbar_arrive_expect_tx(&v_full[st], 16384);
          tma_load_4d(Vs + st * 16384, &tv, &v_full[st], 0, j * 128, h, b);
        }
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    {  // whole warp, converged: the MMA / commit helpers elect the issuing lane
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, D, 0, 1);
      int g0 = 0;            // ring position of this item's first key block
      int cx[2] = {0, 0};    // blocks processed so far per query tile (barrier phase counters)
      int it[2] = {0, 0};    // items in which the tile had blocks (phase of o_empty)
      for (int rnd = 0; rnd * G < n_items; ++rnd) {
        const int w = snake(rnd);
        if (w >= n_items) break;
        const int item = rnd;
        int qp, bh, n_x[2];
        decode(w, qp, bh, n_x[0], n_x[1]);
        const int n_kv = max(n_x[0], n_x[1]);
        mbar_wait(q_full, item & 1, wctx, STATUS_TIMEOUT_PIPE_FULL);
        auto issue_s = [&](int x, int j) {
          const int g = g0 + j;
          mbar_wait(&k_full[g % KS], (g / KS) & 1, wctx, STATUS_TIMEOUT_PIPE_FULL);
          tc_fence_after();
          mma_kk<D / 16>(tmem_base + S_COL + x * 128, smem_u32(Qs + x * 16384), 0, smem_u32(Ks + (g % KS) * 16384),
                         0, idesc_s, false);
          umma_commit_e(&s_full[x]);
        };
        // S(0) of this item may only overwrite S once the softmax has consumed the previous
        // item's last block of that tile; that is guaranteed because the previous item's last
        // P V of the tile was issued after its p_full, and we issue in program order.
        if (n_x[0] > 0) issue_s(0, 0);
        if (n_x[1] > 0) issue_s(1, 0);
        if (n_kv > 0) umma_commit_e(&k_empty[g0 % KS]);
        if (n_kv == 1) umma_commit_e(q_empty);
        // Event loop over both query tiles. Two kinds of events per tile: "scores read out"
        // (s_free: the softmax warps hold block j's scores in registers) lets S(j+1) be issued
        // into the same columns while the exponentials of block j are still being computed, so
        // the next scores are ready when the softmax gets there; "probabilities stored" (p_full)
        // lets P V(j) be issued. Every wait here is a poll, so a tile that is ahead (bounded by
        // the K/V ring, whose stages are released when both tiles have used a
        // block) never blocks the warp that the other tile needs.
        int s_iss[2] = {n_x[0] > 0 ? 1 : 0, n_x[1] > 0 ? 1 : 0};   // S MMAs issued per tile
        int pv_iss[2] = {0, 0};                                     // P V MMAs issued per tile
        uint32_t spins = 0;
        uint64_t spin_t0 = 0;
        bool dead = false;
        while ((pv_iss[0] < n_x[0] || pv_iss[1] < n_x[1]) && !dead) {
          bool progressed = false;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int ot = x ^ 1;
            const int bn = s_iss[x];          // next block whose S is to be issued
            if (bn > 0 && bn < n_x[x]) {
              const int gb = g0 + bn;
              if (mbar_try_wait(&s_free[x], (cx[x] + bn - 1) & 1) &&
                  mbar_try_wait(&k_full[gb % KS], (gb / KS) & 1)) {
                tc_fence_after();
                mma_kk<D / 16>(tmem_base + S_COL + x * 128, smem_u32(Qs + x * 16384), 0,
                               smem_u32(Ks + (gb % KS) * 16384), 0, idesc_s, false);
                umma_commit_e(&s_full[x]);
                s_iss[x] = bn + 1;
                // the K block is free once both tiles' S MMAs on it have been issued
                if (s_iss[ot] > bn || bn >= n_x[ot]) umma_commit_e(&k_empty[gb % KS]);
                if (s_iss[0] >= n_x[0] && s_iss[1] >= n_x[1]) umma_commit_e(q_empty);   // the item's last S
                progressed = true;
              }
            }
            const int j = pv_iss[x];
            if (j < n_x[x]) {
              const int c = cx[x] + j;
              const int g = g0 + j;
              if (mbar_try_wait(&p_full[x], c & 1) && mbar_try_wait(&v_full[g % KS], (g / KS) & 1)) {
                // the accumulator is overwritten once per item: wait until the softmax warps
                // have read the previous item's result out of it
                if (j == 0) mbar_wait(&o_empty[x], (it[x] & 1) ^ 1u, wctx, STATUS_TIMEOUT_SOFTMAX);
                tc_fence_after();
                mma_tmn<8>(tmem_base + OP_COL + x * 64, tmem_base + P_COL + x * 64, smem_u32(Vs + (g % KS) * 16384),
                           0, idesc_o, j > 0);
                umma_commit_e(&o_full[x]);
                pv_iss[x] = j + 1;
                if (pv_iss[ot] > j || j >= n_x[ot]) umma_commit_e(&v_empty[g % KS]);
                progressed = true;
              }
            }
          }
          if (progressed) {
            spins = 0;
            spin_t0 = 0;
          } else if (((++spins) & 0xfffu) == 0u) {
            // bounded like mbar_wait: give up (status recorded) when nothing becomes ready in time
            if (*abort_flag) {
              dead = true;
            } else {
              const uint64_t now = globaltimer_ns();
              if (spin_t0 == 0) {
                spin_t0 = now;
              } else if (now - spin_t0 > GFS_WAIT_LIMIT_NS) {
                *abort_flag = 1u;
                record_status(p.status, STATUS_TIMEOUT_SOFTMAX, (blockIdx.x << 8) | 0xE1u);
                dead = true;
              }
            }
          }
        }
        g0 += n_kv;
        cx[0] += n_x[0];
        cx[1] += n_x[1];
        it[0] += n_x[0] > 0;
        it[1] += n_x[1] > 0;
      }
    }
  } else {
    const int x = (warp - 2) >> 2;           // query tile of this warp
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + S_COL + x * 128;
    const uint32_t o_addr = tmem_base + lane_base + OP_COL + x * 64;
    const uint32_t p_addr = tmem_base + lane_base + P_COL + x * 64;
    const float sl2 = p.scale * LOG2E_F;
    int cdone = 0;  // blocks of this tile processed in earlier items
    {
      for (int rnd = 0; rnd * G < n_items; ++rnd) {
        const int w = snake(rnd);
        if (w >= n_items) break;
        int qp, bh, na, nbk;
        decode(w, qp, bh, na, nbk);
        const int b = bh / p.nh, h = bh % p.nh;
        const int qtx = 2 * qp + x;
        const int row_g = qtx * 128 + r;
        const int n_mine = x == 0 ? na : nbk;
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < n_mine; ++j) {
          const int c = cdone + j;
          const bool need_mask = (p.causal && j == qtx) || ((j + 1) * 128 > p.S);
          mbar_wait(&s_full[x], c & 1, wctx, STATUS_TIMEOUT_SOFTMAX);
          tc_fence_after();
          uint32_t v0[32], v1[32], v2[32], v3[32];
          tmem_ld_32x32(s_addr + 0, v0);
          tmem_ld_32x32(s_addr + 32, v1);
          tmem_ld_32x32(s_addr + 64, v2);
          tmem_ld_32x32(s_addr + 96, v3);
          float mx0 = -INFINITY, mx1 = -INFINITY;
          tmem_ld_wait_for(v0);
          tmem_ld_wait_for(v1);
          tmem_ld_wait_for(v2);
          tmem_ld_wait_for(v3);
          // all 128 scores are in registers: the MMA warp may overwrite S with the next block's
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_free[x]);
          if (need_mask) {
            // Diagonal block (causal) or the block that crosses the end of the sequence: dead scores
            // become -inf in the registers, then the block takes the same code as every other one
            // (exp2(-inf) = 0, max ignores -inf). A separate masked copy of the max / exponential code
            // ran once per work item from a cold instruction cache: 6500 cycles for that block
            // against 2450 for an unmasked one.
            auto mask_chunk = [&](uint32_t (&v)[32], int cc) {
              const int lim_c = p.causal ? row_g - j * 128 - cc : 0x7fffffff;   // last live column of the chunk
              const int lim = min(lim_c, p.S - 1 - j * 128 - cc);
#pragma unroll
              for (int e = 0; e < 32; ++e) v[e] = (e > lim) ? 0xff800000u : v[e];
            };
            mask_chunk(v0, 0);
            mask_chunk(v1, 32);
            mask_chunk(v2, 64);
            mask_chunk(v3, 96);
          }
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            mx0 = fmax3(mx0, __uint_as_float(v0[e]), __uint_as_float(v0[e + 1]));
            mx1 = fmax3(mx1, __uint_as_float(v1[e]), __uint_as_float(v1[e + 1]));
            mx0 = fmax3(mx0, __uint_as_float(v2[e]), __uint_as_float(v2[e + 1]));
            mx1 = fmax3(mx1, __uint_as_float(v3[e]), __uint_as_float(v3[e + 1]));
          }
          const float m_new = fmaxf(m, fmaxf(mx0, mx1));
          // raise the running maximum only when it grew by more than 2^8 (or was still -inf)
          bool grow = false;
          float alpha = 1.f;
          if (m_new > m && (m == -INFINITY || (m_new - m) * sl2 > 8.f)) {
            grow = true;
            alpha = (m == -INFINITY) ? 0.f : fast_exp2((m - m_new) * sl2);
          }
          if (j > 0 && __any_sync(0xffffffffu, grow)) {
            // rescale this warp's 32 accumulator rows in tensor memory (warp-collective accesses;
            // rows whose maximum stays get factor 1). P V of the previous block must be done.
            mbar_wait(&o_full[x], (c - 1) & 1, wctx, STATUS_TIMEOUT_SOFTMAX);
            tc_fence_after();
            const float a = grow ? alpha : 1.f;
#pragma unroll 1
            for (int cc = 0; cc < D; cc += 16) {
              uint32_t wv[16];
              tmem_ld_32x16(o_addr + cc, wv);
              tmem_ld_wait_for16(wv);
#pragma unroll
              for (int e = 0; e < 16; ++e) wv[e] = __float_as_uint(__uint_as_float(wv[e]) * a);
              tmem_st_32x16(o_addr + cc, wv);
            }
            tmem_st_wait();
          }
          if (grow) {
            l *= alpha;
            m = m_new;
          }
          const float moff = ((m == -INFINITY) ? 0.f : m) * sl2;
          float rs0 = 0.f, rs1 = 0.f;
          auto prob_chunk = [&](const uint32_t (&v)[32], uint32_t (&packed)[16]) {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float x0 = fast_exp2(fmaf(__uint_as_float(v[e]), sl2, -moff));
              const float x1 = fast_exp2(fmaf(__uint_as_float(v[e + 1]), sl2, -moff));
              rs0 += x0;
              rs1 += x1;
              packed[e >> 1] = pack_bf16x2(x0, x1);
            }
          };
          uint32_t p0[16], p1[16], p2[16], p3[16];
          prob_chunk(v0, p0);
          prob_chunk(v1, p1);
          prob_chunk(v2, p2);
          prob_chunk(v3, p3);
          l += rs0 + rs1;
          // P of the previous block is read by its P V MMA: overwrite it only when that is done
          if (j > 0) {
            mbar_wait(&o_full[x], (c - 1) & 1, wctx, STATUS_TIMEOUT_SOFTMAX);
            tc_fence_after();
          }
          tmem_st_32x16(p_addr + 0, p0);
          tmem_st_32x16(p_addr + 16, p1);
          tmem_st_32x16(p_addr + 32, p2);
          tmem_st_32x16(p_addr + 48, p3);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[x]);
        }
        if (n_mine > 0) {
          mbar_wait(&o_full[x], (cdone + n_mine - 1) & 1, wctx, STATUS_TIMEOUT_SOFTMAX);
          tc_fence_after();
          uint32_t wa[32], wb[32];
          tmem_ld_32x32(o_addr, wa);
          tmem_ld_32x32(o_addr + 32, wb);
          tmem_ld_wait_for(wa);
          tmem_ld_wait_for(wb);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_empty[x]);   // the next item's first P V may overwrite the accumulator
          const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
          if (row_g < p.S) {
            __nv_bfloat16* dst = p.O + row_g * p.o_ss + b * p.o_bs + h * p.o_hs;
#pragma unroll
            for (int cc = 0; cc < 32; cc += 8) {
              uint4 wv;
              wv.x = pack_bf16x2(__uint_as_float(wa[cc + 0]) * inv_l, __uint_as_float(wa[cc + 1]) * inv_l);
              wv.y = pack_bf16x2(__uint_as_float(wa[cc + 2]) * inv_l, __uint_as_float(wa[cc + 3]) * inv_l);
              wv.z = pack_bf16x2(__uint_as_float(wa[cc + 4]) * inv_l, __uint_as_float(wa[cc + 5]) * inv_l);
              wv.w = pack_bf16x2(__uint_as_float(wa[cc + 6]) * inv_l, __uint_as_float(wa[cc + 7]) * inv_l);
              *reinterpret_cast<uint4*>(dst + cc) = wv;
              wv.x = pack_bf16x2(__uint_as_float(wb[cc + 0]) * inv_l, __uint_as_float(wb[cc + 1]) * inv_l);
              wv.y = pack_bf16x2(__uint_as_float(wb[cc + 2]) * inv_l, __uint_as_float(wb[cc + 3]) * inv_l);
              wv.z = pack_bf16x2(__uint_as_float(wb[cc + 4]) * inv_l, __uint_as_float(wb[cc + 5]) * inv_l);
              wv.w = pack_bf16x2(__uint_as_float(wb[cc + 6]) * inv_l, __uint_as_float(wb[cc + 7]) * inv_l);
              *reinterpret_cast<uint4*>(dst + 32 + cc) = wv;
            }
          }
          if (row_g < p.S_pad) {
            const float mm = (m == -INFINITY) ? 0.f : m;
            p.lse[static_cast<size_t>(bh) * p.S_pad + row_g] = mm * p.scale + logf(fmaxf(l, 1e-37f));
          }
        }
        cdone += n_mine;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// Backward pre-pass: dvec[b,h,s] = sum_d dO[s,b,h,d] * O[s,b,h,d]; one warp per row. Also writes
// lse2 = lse * log2(e), the form the backward's exp2 wants (saves a multiply per score there).
// ---------------------------------------------------------------------------
__global__ void attn_dvec_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                 float* __restrict__ dvec, const float* __restrict__ lse, float* __restrict__ lse2,
                                 int S, int S_pad, int B, int nh, int D, long long do_ss,
                                 long long do_bs, long long do_hs, long long o_ss, long long o_bs, long long o_hs) {
  pdl_wait();
  pdl_trigger();
  // D/8 threads per (s, b, h) row, 16-byte loads; rows ordered h fastest (memory order of [S,B,nh,D]).
  const int tpr = D >> 3;                       // 8 or 16 threads per row
  const int rows_per_block = blockDim.x / tpr;
  const long long row = blockIdx.x * static_cast<long long>(rows_per_block) + threadIdx.x / tpr;
  const int sub = threadIdx.x % tpr;
  const long long total = static_cast<long long>(S) * B * nh;
  float acc = 0.f;
  int h = 0, b = 0, s = 0;
  if (row < total) {
    h = static_cast<int>(row % nh);
    b = static_cast<int>((row / nh) % B);
    s = static_cast<int>(row / (static_cast<long long>(nh) * B));
    const uint4 x = *reinterpret_cast<const uint4*>(dO + s * do_ss + b * do_bs + h * do_hs + sub * 8);
    const uint4 y = *reinterpret_cast<const uint4*>(O + s * o_ss + b * o_bs + h * o_hs + sub * 8);
    const float2 x0 = unpack_bf16x2(x.x), x1 = unpack_bf16x2(x.y), x2 = unpack_bf16x2(x.z), x3 = unpack_bf16x2(x.w);
    const float2 y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y), y2 = unpack_bf16x2(y.z), y3 = unpack_bf16x2(y.w);
    acc = x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y + x2.x * y2.x + x2.y * y2.y + x3.x * y3.x +
          x3.y * y3.y;
  }
  for (int o = tpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (row < total && sub == 0) dvec[(static_cast<size_t>(b) * nh + h) * S_pad + s] = acc;
  // rows S .. S_pad-1 of every head: zeros (the backward multiplies them by probabilities that are 0)
  const int pad = S_pad - S;
  const long long pad_total = static_cast<long long>(pad) * B * nh;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pad_total;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dvec[(i / pad) * S_pad + S + (i % pad)] = 0.f;
  const long long n_lse = static_cast<long long>(S_pad) * B * nh;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_lse;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    lse2[i] = lse[i] * LOG2E_F;
}

// ---------------------------------------------------------------------------
// Backward main kernel
// ---------------------------------------------------------------------------
struct BwdParams {
  __nv_bfloat16* out1;  // mode 0: dK, mode 1: dQ
  __nv_bfloat16* out2;  // mode 0: dV
  long long o1_ss, o1_bs, o1_hs;
  long long o2_ss, o2_bs, o2_hs;
  const float* lse;   // [B, nh, S_pad], already multiplied by log2(e)
  const float* dvec;  // [B, nh, S_pad]
  int S, S_pad, B, nh;
  float scale;
  int causal;
  uint32_t* status;
  // optional: inverse rotary embedding applied to dQ and dK rows before they are stored
  const float* rope_cos;
  const float* rope_sin;
};

// CW = number of compute warps (4 or 8). With 8, every accumulator row is shared by two
// threads that each take half of the 64 streamed columns (no exchange is needed: the
// row/column statistics are inputs), which doubles the warps available to hide latency.
// TS = stages of the streamed-tile ring. A stage is only released when the gradient MMAs that read
// it have finished, and the score MMAs run two tiles ahead, so the TMA of a tile has (TS - 2) tile
// periods to land. head_dim 64 (P / dS in tensor memory, so the shared memory is free) uses 8
// stages: 214 us against 224 us with 4 for the whole backward at the GPT-124M shape, 217 us with
// 10; head_dim 128 has room for 3.
// PP ("ping-pong", needs CW = 8 and NBUF = 2): the two groups of four compute warps take alternate
// streamed tiles (group = X/Y buffer) with all 64 columns per thread instead of column halves of the
// same tile, so that one group's barrier tests, tensor-memory loads and stores overlap the other
// group's arithmetic; and the MMAs are issued by TWO warps (warp 1: scores, warp 2: gradients),
// because a single issuing warp needs ~ 1,350 cycles per tile in that scheme and the compute warps
// then wait for scores.
template <int D, int MODE, int NBUF, int CW, int TS, bool PP>
__global__ void __launch_bounds__((PP ? 96 : 64) + 32 * CW, NBUF == 1 ? 2 : 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tr1, const __grid_constant__ CUtensorMap tr2,
                 const __grid_constant__ CUtensorMap tt1, const __grid_constant__ CUtensorMap tt2,
                 const BwdParams p, int n_rt, int n_items) {
  constexpr int DB = D / 64;
  constexpr int R_BYTES = DB * 16384;  // resident [128 x D]
  constexpr int T_BYTES = DB * 8192;   // streamed [64 x D]
  constexpr int M_BYTES = 16384;       // [128 x 64] bf16
  constexpr uint32_t TMEM_COLS = (NBUF == 1 && D == 64) ? 256 : 512;
  constexpr uint32_t Y_COL = 64 * NBUF;  // X tiles at [0, 64*NBUF), Y tiles after them
  constexpr uint32_t ACC1 = 128 * NBUF, ACC2 = 128 * NBUF + D;
  // head_dim 64 leaves 128 TMEM columns free: P^T / dS^T (bf16, two per column) are handed to the
  // gradient MMAs through tensor memory instead of shared memory, which halves the shared-memory
  // traffic of this kernel (its 64-wide MMAs are otherwise bound by operand reads from shared memory)
  constexpr bool PT = (D == 64 && NBUF == 2);
  constexpr uint32_t PT_COL = 384;  // [buffer][P 32 cols | dS 32 cols]
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  uint8_t* R1 = smem;
  uint8_t* R2 = R1 + R_BYTES;
  uint8_t* T1 = R2 + R_BYTES;        // 2 stages
  uint8_t* T2 = T1 + TS * T_BYTES;
  uint8_t* M1 = T2 + TS * T_BYTES;
  // P / dS through tensor memory: M1 is only the 16 KB staging area of the epilogue, M2 is not used
  uint8_t* M2 = M1 + (PT ? M_BYTES : NBUF * M_BYTES);
  float* stats = reinterpret_cast<float*>(M2 + (PT ? 0 : NBUF * M_BYTES));  // mode 0: [TS stages][lse 64 | dvec 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(stats) + TS * 512);
  uint64_t* r_full = bars;
  uint64_t* t_full = bars + 1;             // [TS]
  uint64_t* t_empty = t_full + TS;         // [TS]
  uint64_t* xy_full = t_empty + TS;
  uint64_t* xy_empty = xy_full + 2;
  uint64_t* m_full = xy_empty + 2;
  uint64_t* m_empty = m_full + 2;
  uint64_t* acc_full = m_empty + 2;
  uint64_t* acc_empty = acc_full + 1;
  uint64_t* r_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 3);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_small = (p.S + 63) >> 6;  // number of 64-row streamed tiles in the sequence
  const int BH = p.B * p.nh;
  // Persistent: a CTA walks work items (resident tile, batch*head), heaviest resident tiles
  // first, dealt in a snake over the CTAs; barrier phases run on counters that continue
  // across items, so set-up and the TMEM allocation are paid once and the next item's loads
  // and first score MMAs overlap the current item's epilogue.
  const int G = static_cast<int>(gridDim.x);
  auto snake = [&](int rnd) {
    return rnd * G + ((rnd & 1) ? G - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x));
  };
  // resident tile index and range of streamed tiles of work item w
  auto decode = [&](int w, int& rt, int& bh, int& t_begin, int& n_t) {
    const int level = w / BH;
    bh = w % BH;
    int t_end;
    if (MODE == 0) {
      rt = level;  // key tile; the first ones have the most query tiles
      t_begin = p.causal ? 2 * rt : 0;
      t_end = n_small;
    } else {
      rt = n_rt - 1 - level;  // query tile; the last ones have the most key tiles
      t_begin = 0;
      t_end = p.causal ? min(n_small, 2 * rt + 2) : n_small;
    }
    n_t = max(t_end - t_begin, 0);
  };

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int i = 0; i < TS; ++i) {
      mbar_init(&t_full[i], 1);
      mbar_init(&t_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&xy_full[i], 1);
      mbar_init(&xy_empty[i], PP ? 4 : CW);
      mbar_init(&m_full[i], PP ? 4 : CW);
      mbar_init(&m_empty[i], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, CW);
    mbar_init(r_empty, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tr1);
    tma_prefetch_desc(&tr2);
    tma_prefetch_desc(&tt1);
    tma_prefetch_desc(&tt2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();       // set-up above may overlap the tail of the preceding kernel (programmatic launch)
  pdl_trigger();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wctx{abort_flag, p.status, GFS_WAIT_LIMIT_NS};

  if (warp == 0) {
    if (lane == 0) {
      int g = 0;  // streamed tiles loaded so far (ring position)
      for (int it = 0; it * G < n_items; ++it) {
        const int w = snake(it);
        if (w >= n_items) break;
        int rt, bh, t_begin, n_t;
        decode(w, rt, bh, t_begin, n_t);
        const int b = bh / p.nh, h = bh % p.nh;
        mbar_wait(r_empty, (it & 1) ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);  // previous item's score MMAs done
      mbar_arrive_expect_tx(r_full, 2 * R_BYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_load_4d(R1 + db * 16384, &tr1, r_full, db * 64, rt * 128, h, b);
        tma_load_4d(R2 + db * 16384, &tr2, r_full, db * 64, rt * 128, h, b);
      }
      for (int t = 0; t < n_t; ++t, ++g) {
        const int st = g % TS;
        const int ti = t_begin + t;
        mbar_wait(&t_empty[st], ((g / TS) & 1) ^ 1u, wctx, STATUS_TIMEOUT_PIPE_EMPTY);
        mbar_arrive_expect_tx(&t_full[st], 2 * T_BYTES + (MODE == 0 ? 512 : 0));
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_4d(T1 + st * T_BYTES + db * 8192, &tt1, &t_full[st], db * 64, ti * 64, h, b);
          tma_load_4d(T2 + st * T_BYTES + db * 8192, &tt2, &t_full[st], db * 64, ti * 64, h, b);
        }
        if (MODE == 0) {
          const size_t off = static_cast<size_t>(bh) * p.S_pad + ti * 64;
          bulk_load_1d(stats + st * 128, p.lse + off, 256, &t_full[st]);
          bulk_load_1d(stats + st * 128 + 64, p.dvec + off, 256, &t_full[st]);
        }
      }
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1 || (PP && warp == 2)) {
    {  // whole warp, converged: the MMA / commit helpers elect the issuing lane
      static_assert(!PP || (CW == 8 && NBUF == 2), "ping-pong needs two warp groups and two X/Y buffers");
      const bool do_xy = !PP || warp == 1;      // this warp issues the score MMAs
      constexpr uint32_t idesc_xy = umma_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, 0, 1);
      const uint32_t r1 = smem_u32(R1), r2 = smem_u32(R2);
      int g0 = 0;  // ring position of the item's first streamed tile
      for (int it = 0; it * G < n_items; ++it) {
        const int w = snake(it);
        if (w >= n_items) break;
        int rt, bh, t_begin, n_t;
        decode(w, rt, bh, t_begin, n_t);
      if (do_xy) mbar_wait(r_full, it & 1, wctx, STATUS_TIMEOUT_PIPE_FULL);
      auto issue_xy = [&](int t) {
        const int g = g0 + t;
        const int st = g % TS;                      // streamed-tile stage
        const uint32_t par = (g / TS) & 1;
        const int sb = (NBUF == 2) ? (g & 1) : 0;   // X / Y / P / dS buffer
        const uint32_t spar = (NBUF == 2) ? ((g >> 1) & 1) : (g & 1);
        mbar_wait(&t_full[st], par, wctx, STATUS_TIMEOUT_PIPE_FULL);
        mbar_wait(&xy_empty[sb], spar ^ 1u, wctx, STATUS_TIMEOUT_SOFTMAX);
        tc_fence_after();
        mma_kk<D / 16>(tmem_base + sb * 64, r1, 16384, smem_u32(T1 + st * T_BYTES), 8192, idesc_xy, false);
        mma_kk<D / 16>(tmem_base + Y_COL + sb * 64, r2, 16384, smem_u32(T2 + st * T_BYTES), 8192, idesc_xy, false);
        umma_commit_e(&xy_full[sb]);
      };
      // Score MMAs run LA blocks ahead of the gradient MMAs. With two X/Y buffers and a ring
      // deep enough (LA = 2), block t+2's scores are issued as soon as the compute warps have
      // pulled block t's X/Y into registers (xy_empty is signalled right after those loads),
      // i.e. while they are still doing block t's math, so they never wait for scores.
      constexpr int LA = (NBUF == 2 && TS >= 4) ? 2 : 1;
      if (PP && do_xy) {
        // score warp: runs ahead as far as the X/Y buffers and the streamed-tile ring allow
        for (int t = 0; t < n_t; ++t) issue_xy(t);
        umma_commit_e(r_empty);
        g0 += n_t;
        continue;
      }
      if (!PP) {
        for (int t = 0; t < LA && t < n_t; ++t) issue_xy(t);
        if (n_t <= LA) umma_commit_e(r_empty);
      }
      for (int t = 0; t < n_t; ++t) {
        if (!PP && t + LA < n_t) {
          issue_xy(t + LA);
          if (t + LA + 1 == n_t) umma_commit_e(r_empty);  // the item's last score MMAs are issued
        }
        const int g = g0 + t;
        const int st = g % TS;
        const int sb = (NBUF == 2) ? (g & 1) : 0;
        mbar_wait(&m_full[sb], (NBUF == 2) ? ((g >> 1) & 1) : (g & 1), wctx, STATUS_TIMEOUT_SOFTMAX);
        if (t == 0) mbar_wait(acc_empty, (it & 1) ^ 1u, wctx, STATUS_TIMEOUT_TMEM_EMPTY);  // previous epilogue done
        tc_fence_after();
        if (PT) {
          const uint32_t pt = tmem_base + PT_COL + sb * 64;
          if (MODE == 0) {
            mma_tmn<4>(tmem_base + ACC1, pt, smem_u32(T2 + st * T_BYTES), 8192, idesc_acc, t > 0);        // dV += P^T dO
            mma_tmn<4>(tmem_base + ACC2, pt + 32, smem_u32(T1 + st * T_BYTES), 8192, idesc_acc, t > 0);   // dK += dS^T Q
          } else {
            mma_tmn<4>(tmem_base + ACC1, pt + 32, smem_u32(T1 + st * T_BYTES), 8192, idesc_acc, t > 0);   // dQ += dS K
          }
        } else if (MODE == 0) {
          // dV += P^T dO ; dK += dS^T Q
          mma_kmn<4>(tmem_base + ACC1, smem_u32(M1 + sb * M_BYTES), 0, smem_u32(T2 + st * T_BYTES), 8192, idesc_acc,
                     t > 0);
          mma_kmn<4>(tmem_base + ACC2, smem_u32(M2 + sb * M_BYTES), 0, smem_u32(T1 + st * T_BYTES), 8192, idesc_acc,
                     t > 0);
        } else {
          // dQ += dS K
          mma_kmn<4>(tmem_base + ACC1, smem_u32(M1 + sb * M_BYTES), 0, smem_u32(T1 + st * T_BYTES), 8192, idesc_acc,
                     t > 0);
        }
        umma_commit_e(&t_empty[st]);
        umma_commit_e(&m_empty[sb]);
      }
      umma_commit_e(acc_full);
      g0 += n_t;
      }
    }
  } else {
    const int quarter = warp & 3;
    constexpr int FIRST_CW = PP ? 3 : 2;            // first compute warp
    constexpr int COLS = PP ? 64 : 64 / (CW / 4);   // streamed columns handled by this thread
    const int chalf = (CW == 8) ? ((warp - FIRST_CW) >> 2) : 0;   // warp group: epilogue column half; tile parity (PP) or column half of the math
    const int cbase = PP ? 0 : chalf * COLS;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale * LOG2E_F;
    int g0 = 0;
    for (int it = 0; it * G < n_items; ++it) {
    const int w = snake(it);
    if (w >= n_items) break;
    int rt, bh, t_begin, n_t;
    decode(w, rt, bh, t_begin, n_t);
    const int b = bh / p.nh, h = bh % p.nh;
    const int row_g = rt * 128 + r;  // mode 0: key position, mode 1: query position
    float row_lse = 0.f, row_dvec = 0.f;
    if (MODE == 1 && row_g < p.S_pad) {
      row_lse = p.lse[static_cast<size_t>(bh) * p.S_pad + row_g];
      row_dvec = p.dvec[static_cast<size_t>(bh) * p.S_pad + row_g];
    }
    for (int t = 0; t < n_t; ++t) {
      const int g = g0 + t;
      const int st = g % TS;                      // streamed-tile stage (for the column statistics)
      const int sb = (NBUF == 2) ? (g & 1) : 0;   // X / Y / P / dS buffer
      const uint32_t par = (NBUF == 2) ? ((g >> 1) & 1) : (g & 1);
      if (PP && sb != chalf) continue;            // the other warp group's tile
      const int ti = t_begin + t;
      bool need_mask;
      if (MODE == 0) need_mask = (p.causal && ti < 2 * rt + 2) || ((ti + 1) * 64 > p.S);
      else need_mask = (p.causal && ti >= 2 * rt) || ((ti + 1) * 64 > p.S);
      mbar_wait(&xy_full[sb], par, wctx, STATUS_TIMEOUT_SOFTMAX);
      mbar_wait(&m_empty[sb], par ^ 1u, wctx, STATUS_TIMEOUT_SOFTMAX);
      tc_fence_after();
      const float* st_lse = stats + st * 128;
      const float* st_dv = st_lse + 64;
      uint8_t* m1row = M1 + sb * M_BYTES + r * 128;
      uint8_t* m2row = M2 + sb * M_BYTES + r * 128;
      uint32_t xa[32], ya[32], xb[32], yb[32];
      // Masked tiles (the diagonal, the sequence tail) turn their dead scores into -inf in the
      // registers, which makes both P and dS exact zeros (dvec and dP are finite everywhere, the
      // padding rows of dvec are written as zeros), and then run the same code as every other tile.
      auto grad_chunk_impl = [&](uint32_t (&xv)[32], const uint32_t (&yv)[32], int c) {
        if (need_mask) {
          const int col0 = ti * 64 + c;
          const int hi = p.S - col0;                                   // first column past the sequence
          if (MODE == 0) {                                             // col = query, row = key
            const int lo = p.causal ? row_g - col0 : -0x7fffffff;      // queries before the key are dead
#pragma unroll
            for (int e = 0; e < 32; ++e) xv[e] = (e < lo || e >= hi) ? 0xff800000u : xv[e];
          } else {                                                     // col = key, row = query
            const int lim = min(p.causal ? row_g - col0 : 0x7fffffff, hi - 1);
#pragma unroll
            for (int e = 0; e < 32; ++e) xv[e] = (e > lim) ? 0xff800000u : xv[e];
          }
        }
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          float ls[4], dv[4];
          if (MODE == 0) {   // per-column statistics of the streamed query tile (same address in all lanes)
            const float4 l4 = *reinterpret_cast<const float4*>(st_lse + c + e);
            const float4 d4 = *reinterpret_cast<const float4*>(st_dv + c + e);
            ls[0] = l4.x; ls[1] = l4.y; ls[2] = l4.z; ls[3] = l4.w;
            dv[0] = d4.x; dv[1] = d4.y; dv[2] = d4.z; dv[3] = d4.w;
          } else {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              ls[u] = row_lse;
              dv[u] = row_dvec;
            }
          }
          float pe[4], de[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            pe[u] = fast_exp2(fmaf(__uint_as_float(xv[e + u]), sl2, -ls[u]));
            de[u] = pe[u] * (__uint_as_float(yv[e + u]) - dv[u]);
          }
          if (MODE == 0) {
            pp[e >> 1] = pack_bf16x2(pe[0], pe[1]);
            pp[(e >> 1) + 1] = pack_bf16x2(pe[2], pe[3]);
          }
          dd[e >> 1] = pack_bf16x2(de[0], de[1]);
          dd[(e >> 1) + 1] = pack_bf16x2(de[2], de[3]);
        }
        if (PT) {
          // columns c .. c+31 of this row -> 16 packed columns of the P / dS tensor-memory tiles
          const uint32_t pt = tmem_base + lane_base + PT_COL + sb * 64 + (c >> 1);
          if (MODE == 0) tmem_st_32x16(pt, pp);
          tmem_st_32x16(pt + 32, dd);
          return;
        }
        const int chunk0 = c >> 3;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int off = (((chunk0 + q4) ^ (r & 7)) & 7) << 4;
          if (MODE == 0) {
            *reinterpret_cast<uint4*>(m1row + off) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2],
                                                                 pp[4 * q4 + 3]);
          }
          *reinterpret_cast<uint4*>((MODE == 0 ? m2row : m1row) + off) =
              make_uint4(dd[4 * q4], dd[4 * q4 + 1], dd[4 * q4 + 2], dd[4 * q4 + 3]);
        }
      };
      auto grad_chunk = [&](uint32_t (&xv)[32], const uint32_t (&yv)[32], int c) {
        // alive / mixed / dead for this warp's 32 rows x 32 columns; a dead chunk costs no math
        const int row_lo = rt * 128 + quarter * 32;
        const int kind = need_mask ? mask_class<MODE == 0>(row_lo, row_lo + 31, ti * 64 + c, ti * 64 + c + 31,
                                                           p.causal != 0, p.S)
                                   : 0;
        if (kind == 2 && PT) {
          uint32_t zeros[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) zeros[e] = 0u;
          const uint32_t pt = tmem_base + lane_base + PT_COL + sb * 64 + (c >> 1);
          if (MODE == 0) tmem_st_32x16(pt, zeros);
          tmem_st_32x16(pt + 32, zeros);
        } else {
          grad_chunk_impl(xv, yv, c);
        }
      };
      const uint32_t x_addr = tmem_base + lane_base + sb * 64;
      const uint32_t y_addr = tmem_base + lane_base + Y_COL + sb * 64;
      if (PP) {
        // one 32-column half at a time in the same registers (all 64 columns at once would not fit
        // the 168 registers of a thread); the X/Y buffer goes back once the second half is loaded
        tmem_ld_32x32(x_addr, xa);
        tmem_ld_32x32(y_addr, ya);
        tmem_ld_wait_for(xa);
        tmem_ld_wait_for(ya);
        grad_chunk(xa, ya, 0);
        tmem_ld_32x32(x_addr + 32, xa);
        tmem_ld_32x32(y_addr + 32, ya);
        tmem_ld_wait_for(xa);
        tmem_ld_wait_for(ya);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&xy_empty[sb]);
        grad_chunk(xa, ya, 32);
      } else {
        tmem_ld_32x32(x_addr + cbase, xa);
        tmem_ld_32x32(y_addr + cbase, ya);
        if (COLS == 64) {
          tmem_ld_32x32(x_addr + 32, xb);
          tmem_ld_32x32(y_addr + 32, yb);
        }
        tmem_ld_wait_for(xa);
        tmem_ld_wait_for(ya);
        if (COLS == 64) {
          tmem_ld_wait_for(xb);
          tmem_ld_wait_for(yb);
        }
        // X / Y are in registers: hand the buffer back now so the next scores can be computed
        // into it while this block's math runs
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&xy_empty[sb]);
        grad_chunk(xa, ya, cbase);
        if (COLS == 64) grad_chunk(xb, yb, 32);
      }
      if (PT) tmem_st_wait();
      tc_fence_before();
      if (!PT) fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&m_full[sb]);
    }
    // epilogue: accumulators -> global
    g0 += n_t;
    // the rotary table entries of this thread's row and columns are fetched while the item's last
    // gradient MMAs finish (their global-memory latency would otherwise sit between the
    // accumulator load and the stores)
    constexpr int EC = D / (CW / 4);   // accumulator columns per thread
    float4 rope_c[EC / 8], rope_s[EC / 8];
    const bool rope_on = p.rope_cos != nullptr && row_g < p.S;
    if (rope_on) {
#pragma unroll
      for (int i = 0; i < EC / 8; ++i) {
        const size_t ti = static_cast<size_t>(row_g) * (D / 2) + ((chalf * EC + 8 * i) >> 1);
        rope_c[i] = *reinterpret_cast<const float4*>(p.rope_cos + ti);
        rope_s[i] = *reinterpret_cast<const float4*>(p.rope_sin + ti);
      }
    }
    mbar_wait(acc_full, it & 1, wctx, STATUS_TIMEOUT_TMEM_FULL);
    tc_fence_after();
    // The accumulators leave through a staging area in the M1 buffer (nothing reads it any more:
    // acc_full covers the item's last gradient MMAs): rows [32 * quarter, +32) of M1 are only ever
    // written by the two warps of this quarter, which meet at a named barrier before either of them
    // goes on to the next item's first block.
    const int row0 = rt * 128 + quarter * 32;
    uint8_t* stage = M1 + quarter * 4096 + chalf * 2048;
    __nv_bfloat16* g1 = p.out1 + row0 * p.o1_ss + b * p.o1_bs + h * p.o1_hs;
    __nv_bfloat16* g2 = (MODE == 0) ? p.out2 + row0 * p.o2_ss + b * p.o2_bs + h * p.o2_hs : nullptr;
#pragma unroll
    for (int ci = 0; ci < EC / 32; ++ci) {
      const int c = chalf * EC + 32 * ci;
      uint32_t v[32], w[16];
      // mode 0: ACC2 holds dK (scaled), ACC1 holds dV; mode 1: ACC1 holds dQ (scaled)
      tmem_ld_32x32(tmem_base + lane_base + (MODE == 0 ? ACC2 : ACC1) + c, v);
      tmem_ld_wait();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[8 * q4 + e]) * p.scale;
        if (rope_on) {  // inverse rotation: sin -> -sin
          const float4 cs = rope_c[4 * ci + q4];
          const float4 sn = rope_s[4 * ci + q4];
          const float a0 = f[0], a1 = f[1], a2 = f[2], a3 = f[3], a4 = f[4], a5 = f[5], a6 = f[6], a7 = f[7];
          f[0] = a0 * cs.x + a1 * sn.x; f[1] = a1 * cs.x - a0 * sn.x;
          f[2] = a2 * cs.y + a3 * sn.y; f[3] = a3 * cs.y - a2 * sn.y;
          f[4] = a4 * cs.z + a5 * sn.z; f[5] = a5 * cs.z - a4 * sn.z;
          f[6] = a6 * cs.w + a7 * sn.w; f[7] = a7 * cs.w - a6 * sn.w;
        }
        w[4 * q4 + 0] = pack_bf16x2(f[0], f[1]);
        w[4 * q4 + 1] = pack_bf16x2(f[2], f[3]);
        w[4 * q4 + 2] = pack_bf16x2(f[4], f[5]);
        w[4 * q4 + 3] = pack_bf16x2(f[6], f[7]);
      }
      store_rows_32x32(stage, w, lane, g1 + c, p.o1_ss, p.S - row0);
      if (MODE == 0) {
        tmem_ld_32x32(tmem_base + lane_base + ACC1 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) w[e] = pack_bf16x2(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
        store_rows_32x32(stage, w, lane, g2 + c, p.o2_ss, p.S - row0);
      }
    }
    if (CW == 8) named_barrier_sync(8 + quarter, 64);
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(acc_empty);  // the accumulators may be overwritten by the next item
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

const CUtensorMap* make_map(const void* base, int D, int S, int nh, int B, const long long* st, uint32_t box_rows) {
  // st = {seq, batch, head} element strides
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(nh),
                      static_cast<uint64_t>(B)};
  uint64_t strides[4] = {2, static_cast<uint64_t>(st[0]) * 2, static_cast<uint64_t>(st[2]) * 2,
                         static_cast<uint64_t>(st[1]) * 2};
  uint32_t box[4] = {64, box_rows, 1, 1};
  return gfs_host::tmap_nd_cached(base, 4, dims, strides, box);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -10;
}

bool strides_ok(const long long* st, int n) {
  for (int i = 0; i < n; ++i)
    if (st[i] & 7) return false;
  return true;
}

}  // namespace

extern "C" {

// strides: 12 element strides {q_seq,q_batch,q_head, k_.., v_.., o_..}. lse: fp32 [B, nh, S_pad],
// S_pad = S rounded up to a multiple of 128.
int gfs_flash_fwd(const void* q, const void* k, const void* v, void* o, void* lse, int S, int B, int nh, int D,
                  const long long* strides, float scale, int causal, void* stream_) {
  if (D != 64 && D != 128) return -1;
  if (!strides_ok(strides, 12)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -2;
  if (S <= 0 || B <= 0 || nh <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const CUtensorMap* tq = make_map(q, D, S, nh, B, strides + 0, 128);
  const CUtensorMap* tk = make_map(k, D, S, nh, B, strides + 3, 128);
  const CUtensorMap* tv = make_map(v, D, S, nh, B, strides + 6, 128);
  if (!tq || !tk || !tv) return -3;
  FwdParams p;
  p.O = static_cast<__nv_bfloat16*>(o);
  p.o_ss = strides[9]; p.o_bs = strides[10]; p.o_hs = strides[11];
  p.lse = static_cast<float*>(lse);
  p.S = S; p.S_pad = ((S + 127) / 128) * 128; p.B = B; p.nh = nh;
  p.scale = scale; p.causal = causal;
  p.status = gfs_host::status_words();
  const dim3 grid((S + 127) / 128, B * nh);
  static bool set64 = false, set128 = false;
  if (D == 64) {
    if (!set64) {
      if (set_smem(flash_fwd64_kernel, FWD64_SMEM)) return -10;
      set64 = true;
    }
    const int n_pairs = (static_cast<int>(grid.x) + 1) / 2;
    const int n_items = n_pairs * B * nh;
    const int ctas = std::min(n_items, gfs_host::sm_count());
    gfs_host::launch_pdl(flash_fwd64_kernel, dim3(ctas), dim3(FWD64_THREADS), FWD64_SMEM, stream, *tq, *tk, *tv, p,
                         n_pairs, n_items);
  } else {
    const int smem = 32768 * 5 + 2 * 32768 + 256;
    if (!set128) { if (set_smem(flash_fwd_kernel<128, 2>, smem)) return -10; set128 = true; }
    gfs_host::launch_pdl(flash_fwd_kernel<128, 2>, grid, dim3(ATT_THREADS), smem, stream, *tq, *tk, *tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// strides: 24 element strides for {q, k, v, o, do, dq, dk, dv} x {seq, batch, head}.
// lse, dvec: fp32 [B, nh, S_pad]; dvec is scratch written by the pre-pass.
// rope_cos / rope_sin (optional, fp32 [>=S, D/2]): when given, dq and dk are rotated back
// (inverse rotary embedding) as they are written, i.e. they are gradients w.r.t. the
// un-rotated projections.
int gfs_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dO, const void* lse,
                  void* dvec, void* dq, void* dk, void* dv, int S, int B, int nh, int D, const long long* strides,
                  float scale, int causal, const void* rope_cos, const void* rope_sin, void* stream_) {
  if (D != 64 && D != 128) return -1;
  if (!strides_ok(strides, 24)) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(dO) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
       reinterpret_cast<uintptr_t>(dv)) & 15)
    return -2;
  if (S <= 0 || B <= 0 || nh <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int S_pad = ((S + 127) / 128) * 128;
  const long long *sq = strides, *sk = strides + 3, *sv = strides + 6, *so = strides + 9, *sdo = strides + 12,
                  *sdq = strides + 15, *sdk = strides + 18, *sdv = strides + 21;
  // second half of the dvec buffer: lse * log2(e)
  float* lse2 = static_cast<float*>(dvec) + static_cast<size_t>(S_pad) * B * nh;
  {
    const long long rows = static_cast<long long>(S) * B * nh;
    const int threads = 256;
    const int rows_per_block = threads / (D >> 3);
    gfs_host::launch_pdl(attn_dvec_kernel, dim3(static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block)),
                         dim3(threads), 0, stream, static_cast<const __nv_bfloat16*>(dO),
                         static_cast<const __nv_bfloat16*>(o), static_cast<float*>(dvec),
                         static_cast<const float*>(lse), lse2, S, S_pad, B, nh, D, sdo[0], sdo[1], sdo[2], so[0],
                         so[1], so[2]);
    if (cudaGetLastError() != cudaSuccess) return -11;
  }
  const CUtensorMap* q128 = make_map(q, D, S, nh, B, sq, 128);
  const CUtensorMap* k128 = make_map(k, D, S, nh, B, sk, 128);
  const CUtensorMap* v128 = make_map(v, D, S, nh, B, sv, 128);
  const CUtensorMap* do128 = make_map(dO, D, S, nh, B, sdo, 128);
  const CUtensorMap* q64 = make_map(q, D, S, nh, B, sq, 64);
  const CUtensorMap* k64 = make_map(k, D, S, nh, B, sk, 64);
  const CUtensorMap* v64 = make_map(v, D, S, nh, B, sv, 64);
  const CUtensorMap* do64 = make_map(dO, D, S, nh, B, sdo, 64);
  if (!q128 || !k128 || !v128 || !do128 || !q64 || !k64 || !v64 || !do64) return -3;
  BwdParams p;
  p.lse = lse2;
  p.dvec = static_cast<const float*>(dvec);
  p.S = S; p.S_pad = S_pad; p.B = B; p.nh = nh; p.scale = scale; p.causal = causal;
  p.status = gfs_host::status_words();
  p.rope_cos = static_cast<const float*>(rope_cos);
  p.rope_sin = static_cast<const float*>(rope_sin);
  const int n_rt = (S + 127) / 128;
  const int n_items = n_rt * B * nh;
  const int ctas = std::min(n_items, gfs_host::sm_count());
  const int nbuf = 2;
  const int bwd_threads = ((D == 64) ? 96 : 64) + 32 * 8;   // head_dim 64: a second MMA-issuing warp
  const int ts = (D == 64) ? 8 : 3;
  const int m_bytes = (D == 64) ? 16384 : 2 * nbuf * 16384;   // head_dim 64: epilogue staging only
  const int smem = 2 * (D / 64) * 16384 + 2 * ts * (D / 64) * 8192 + m_bytes + ts * 512 + 512 + 1024;
  static bool set_done[4] = {false, false, false, false};
  // mode 0: dK, dV
  BwdParams p0 = p;
  p0.out1 = static_cast<__nv_bfloat16*>(dk); p0.o1_ss = sdk[0]; p0.o1_bs = sdk[1]; p0.o1_hs = sdk[2];
  p0.out2 = static_cast<__nv_bfloat16*>(dv); p0.o2_ss = sdv[0]; p0.o2_bs = sdv[1]; p0.o2_hs = sdv[2];
  BwdParams p1 = p;
  p1.out1 = static_cast<__nv_bfloat16*>(dq); p1.o1_ss = sdq[0]; p1.o1_bs = sdq[1]; p1.o1_hs = sdq[2];
  p1.out2 = nullptr; p1.o2_ss = p1.o2_bs = p1.o2_hs = 0;
  if (D == 64) {
    if (!set_done[0]) { if (set_smem(flash_bwd_kernel<64, 0, 2, 8, 8, true>, smem)) return -10; set_done[0] = true; }
    if (!set_done[1]) { if (set_smem(flash_bwd_kernel<64, 1, 2, 8, 8, true>, smem)) return -10; set_done[1] = true; }
    gfs_host::launch_pdl(flash_bwd_kernel<64, 0, 2, 8, 8, true>, dim3(ctas), dim3(bwd_threads), smem, stream, *k128, *v128,
                         *q64, *do64, p0, n_rt, n_items);
    if (cudaGetLastError() != cudaSuccess) return -12;
    gfs_host::launch_pdl(flash_bwd_kernel<64, 1, 2, 8, 8, true>, dim3(ctas), dim3(bwd_threads), smem, stream, *q128, *do128,
                         *k64, *v64, p1, n_rt, n_items);
  } else {
    if (!set_done[2]) { if (set_smem(flash_bwd_kernel<128, 0, 2, 8, 3, false>, smem)) return -10; set_done[2] = true; }
    if (!set_done[3]) { if (set_smem(flash_bwd_kernel<128, 1, 2, 8, 3, false>, smem)) return -10; set_done[3] = true; }
    gfs_host::launch_pdl(flash_bwd_kernel<128, 0, 2, 8, 3, false>, dim3(ctas), dim3(bwd_threads), smem, stream, *k128, *v128,
                         *q64, *do64, p0, n_rt, n_items);
    if (cudaGetLastError() != cudaSuccess) return -12;
    gfs_host::launch_pdl(flash_bwd_kernel<128, 1, 2, 8, 3, false>, dim3(ctas), dim3(bwd_threads), smem, stream, *q128, *do128,
                         *k64, *v64, p1, n_rt, n_items);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -13;
}

}  // extern "C"
