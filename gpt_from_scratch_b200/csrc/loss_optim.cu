// Vocab-parallel cross entropy (local part + combine + in-place backward) and the
// fused optimizer kernels (sum of squares, clip + AdamW + bf16 cast).
//
// Reference counterparts: core/tensor_parallel/loss.py:9-72 (ten ATen kernels and two
// extra [S,B,V/P] tensors become one read of the logits forward and one in-place
// read-modify-write backward) and core/optimizer.py:79-104 (cast, square, sum, host-side
// compare, scale, AdamW, cast become two kernels with the clip decided on the device).
#include <algorithm>

#include "common.cuh"

using namespace gfs;

namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

constexpr int CE_THREADS = 256;

// One CTA per row of the local logits [M, Vp] (pitch ld). Online max / sum-exp in a
// single pass. stats[row] = {local max, sum exp(z - max), z[target] or 0 if the target
// id is outside [v0, v0+Vp)}. With single_rank != 0 also writes lse and loss.
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
              float* __restrict__ stats, float* __restrict__ lse, float* __restrict__ loss, int Vp, long ld, int v0,
              int single_rank) {
  const int row = blockIdx.x;
  const __nv_bfloat16* z = logits + static_cast<size_t>(row) * ld;
  const int nvec = Vp >> 3;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    float f[8];
    load8(z + 8 * v, f);
    float vm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) vm = fmaxf(vm, f[e]);
    const float nm = fmaxf(m, vm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += __expf(f[e] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  // combine (m, s) across the CTA
  __shared__ float sm_m[CE_THREADS / 32], sm_s[CE_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float wm = warp_max(m);
  const float ws = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
  if (lane == 0) {
    sm_m[warp] = wm;
    sm_s[warp] = ws;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float gm = sm_m[0];
    for (int i = 1; i < CE_THREADS / 32; ++i) gm = fmaxf(gm, sm_m[i]);
    float gs = 0.f;
    for (int i = 0; i < CE_THREADS / 32; ++i) gs += (sm_m[i] == -INFINITY) ? 0.f : sm_s[i] * __expf(sm_m[i] - gm);
    const long long t = target[row];
    float tz = 0.f;
    if (t >= v0 && t < v0 + Vp) tz = __bfloat162float(z[t - v0]);
    stats[3 * row + 0] = gm;
    stats[3 * row + 1] = gs;
    stats[3 * row + 2] = tz;
    if (single_rank) {
      const float l = gm + __logf(gs);
      lse[row] = l;
      loss[row] = l - tz;
    }
  }
}

// Same outputs as ce_fwd_kernel, from per-slice statistics that the LM-head GEMM epilogue already
// produced (partials: float2 {max, sum exp(x - max)} [parts][M]); only the target logit is read
// from the logits. A block owns 32 consecutive rows (lane = row, so a warp reads 256 contiguous
// bytes per slice); its CE_PW warps split the slices and keep four loads in flight each, then one
// warp merges the per-warp results in a fixed order. (One thread per row walking all slices was a
// chain of dependent loads: ~100 us at 8192 rows x 198 slices for 13 MB of input.)
constexpr int CE_PW = 8;
__device__ __forceinline__ void ce_merge(float& gm, float& gs, float2 ms) {
  const float nm = fmaxf(gm, ms.x);
  if (nm != -INFINITY) gs = gs * __expf(gm - nm) + ms.y * __expf(ms.x - nm);
  gm = nm;
}
__global__ void __launch_bounds__(32 * CE_PW)
ce_from_partials_kernel(const float2* __restrict__ partials, const __nv_bfloat16* __restrict__ logits,
                        const long long* __restrict__ target, float* __restrict__ stats, float* __restrict__ lse,
                        float* __restrict__ loss, int parts, int M, int Vp, long ld, int v0, int single_rank) {
  __shared__ float2 part_res[CE_PW][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * 32 + lane;
  float gm = -INFINITY, gs = 0.f;
  if (row < M) {
    const float2 empty = make_float2(-INFINITY, 0.f);
    for (int i = warp; i < parts; i += 4 * CE_PW) {
      float2 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int pi = i + u * CE_PW;
        v[u] = (pi < parts) ? partials[static_cast<size_t>(pi) * M + row] : empty;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) ce_merge(gm, gs, v[u]);
    }
  }
  part_res[warp][lane] = make_float2(gm, gs);
  __syncthreads();
  if (warp != 0 || row >= M) return;
  gm = -INFINITY;
  gs = 0.f;
#pragma unroll
  for (int w = 0; w < CE_PW; ++w) ce_merge(gm, gs, part_res[w][lane]);
  const long long t = target[row];
  float tz = 0.f;
  if (t >= v0 && t < v0 + Vp) tz = __bfloat162float(logits[static_cast<size_t>(row) * ld + (t - v0)]);
  stats[3 * row + 0] = gm;
  stats[3 * row + 1] = gs;
  stats[3 * row + 2] = tz;
  if (single_rank) {
    const float l = gm + __logf(gs);
    lse[row] = l;
    loss[row] = l - tz;
  }
}

// Combine the per-rank stats of `world` ranks (stats_all is [world, M, 3]).
__global__ void ce_combine_kernel(const float* __restrict__ stats_all, float* __restrict__ lse,
                                  float* __restrict__ loss, int M, int world) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float gm = -INFINITY;
  for (int r = 0; r < world; ++r) gm = fmaxf(gm, stats_all[(static_cast<size_t>(r) * M + row) * 3]);
  float gs = 0.f, tz = 0.f;
  for (int r = 0; r < world; ++r) {
    const float* st = stats_all + (static_cast<size_t>(r) * M + row) * 3;
    gs += st[1] * __expf(st[0] - gm);
    tz += st[2];
  }
  const float l = gm + __logf(gs);
  lse[row] = l;
  loss[row] = l - tz;
}

// In place: z <- (exp(z - lse) - [col == target - v0]) * g[row]. Grid: x covers the vectors of
// a row, y strides over rows.
__global__ void ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, const float* __restrict__ lse,
                              const long long* __restrict__ target, const float* __restrict__ grad_rows, int M, int Vp,
                              long ld, int v0) {
  const int nvec = Vp >> 3;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= nvec) return;
  const int c = v << 3;
  // four rows per iteration, their loads issued together (each thread owns one 16-byte column
  // group; a single row per thread leaves too little in flight to reach memory speed)
  constexpr int U = 4;
  for (int row0 = blockIdx.y * U; row0 < M; row0 += gridDim.y * U) {
    uint4 raw[U];
    float l[U], g[U];
    long long t[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = row0 + u;
      if (row < M) {
        raw[u] = *reinterpret_cast<const uint4*>(logits + static_cast<size_t>(row) * ld + c);
        l[u] = lse[row];
        g[u] = grad_rows[row];
        t[u] = target[row] - v0;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int row = row0 + u;
      if (row >= M) break;
      const float2 a0 = unpack_bf16x2(raw[u].x), a1 = unpack_bf16x2(raw[u].y), a2 = unpack_bf16x2(raw[u].z),
                   a3 = unpack_bf16x2(raw[u].w);
      float f[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float sm = __expf(f[e] - l[u]);
        if (t[u] == c + e) sm -= 1.f;
        f[e] = sm * g[u];
      }
      store8(logits + static_cast<size_t>(row) * ld + c, f);
    }
  }
}

// ---------------------------------------------------------------------------
// Optimizer
// ---------------------------------------------------------------------------
constexpr int SUMSQ_THREADS = 256;
constexpr int SUMSQ_MAX_BLOCKS = 1024;

// Sum of squares of a bf16 vector, deterministic: per-block partials, the last block to
// finish (ticket counter) adds them in index order and writes out[0]. scratch holds
// SUMSQ_MAX_BLOCKS floats followed by one uint32 ticket that must start at zero
// (the kernel resets it).
__global__ void __launch_bounds__(SUMSQ_THREADS)
sumsq_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ out,
                  float* __restrict__ scratch) {
  float acc = 0.f;
  const long long nvec = n >> 3;
  for (long long v = blockIdx.x * static_cast<long long>(SUMSQ_THREADS) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * SUMSQ_THREADS) {
    float f[8];
    load8(x + 8 * v, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
  }
  if (blockIdx.x == 0) {
    for (long long i = (nvec << 3) + threadIdx.x; i < n; i += SUMSQ_THREADS) {
      const float f = __bfloat162float(x[i]);
      acc += f * f;
    }
  }
  __shared__ float sm[SUMSQ_THREADS / 32];
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  acc = warp_sum(acc);
  if (lane == 0) sm[warp] = acc;
  __syncthreads();
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch + SUMSQ_MAX_BLOCKS);
  if (threadIdx.x == 0) {
    float b = 0.f;
    for (int i = 0; i < SUMSQ_THREADS / 32; ++i) b += sm[i];
    scratch[blockIdx.x] = b;
    __threadfence();
    const unsigned int prev = atomicAdd(ticket, 1u);
    is_last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last) {
    // fixed-order parallel sum of the per-block partials (same result on every run)
    __threadfence();
    float t = 0.f;
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += SUMSQ_THREADS)
      t += reinterpret_cast<volatile float*>(scratch)[i];
    t = warp_sum(t);
    __syncthreads();
    if (lane == 0) sm[warp] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int i = 0; i < SUMSQ_THREADS / 32; ++i) total += sm[i];
      out[0] = total;
      *ticket = 0u;
    }
  }
}


// g <- grad * grad_scale * clip_coef (clip_coef from the device scalar *sumsq, which holds the
// squared norm of grad * grad_scale... see launcher), then torch.optim.AdamW's update on the fp32
// master value, and the bf16 cast of the new value into the parameter buffer.
__global__ void adamw_kernel(const __nv_bfloat16* __restrict__ grad, float* __restrict__ master,
                             float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
                             __nv_bfloat16* __restrict__ param_out, long long n, const float* __restrict__ sumsq,
                             float* __restrict__ norm_out, AdamArgs a) {
  float coef = a.grad_scale;
  if (sumsq != nullptr) {
    const float norm = sqrtf(*sumsq) * a.grad_scale;
    if (norm_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *norm_out = norm;
    if (a.clip > 0.f && norm > a.clip) coef *= a.clip / (norm + 1e-6f);
  }
  float bc1, bc2_sqrt;
  adam_bias_corrections(a, bc1, bc2_sqrt);
  const float decay = 1.f - a.lr * a.weight_decay;
  const float step = a.lr / bc1;
  const float ob1 = 1.f - a.beta1, ob2 = 1.f - a.beta2;
  auto update = [&](float g, float& p, float& m, float& v) {
    g *= coef;
    p *= decay;
    m = a.beta1 * m + ob1 * g;
    v = a.beta2 * v + ob2 * g * g;
    p -= step * (m / (sqrtf(v) / bc2_sqrt + a.eps));
  };
  // vector body: 4 elements per thread (8-byte bf16 and 16-byte fp32 accesses); all four
  // arrays are 16-byte aligned slices when n's base offset is a multiple of 4 elements
  const bool aligned = ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(param_out)) & 7) == 0 &&
                       ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(exp_avg) |
                         reinterpret_cast<uintptr_t>(exp_avg_sq)) & 15) == 0;
  const long long nvec = aligned ? (n >> 2) : 0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint2 gr = reinterpret_cast<const uint2*>(grad)[i];
    float4 p = reinterpret_cast<float4*>(master)[i];
    float4 m = reinterpret_cast<float4*>(exp_avg)[i];
    float4 v = reinterpret_cast<float4*>(exp_avg_sq)[i];
    const float2 g01 = unpack_bf16x2(gr.x), g23 = unpack_bf16x2(gr.y);
    update(g01.x, p.x, m.x, v.x);
    update(g01.y, p.y, m.y, v.y);
    update(g23.x, p.z, m.z, v.z);
    update(g23.y, p.w, m.w, v.w);
    reinterpret_cast<float4*>(master)[i] = p;
    reinterpret_cast<float4*>(exp_avg)[i] = m;
    reinterpret_cast<float4*>(exp_avg_sq)[i] = v;
    reinterpret_cast<uint2*>(param_out)[i] = make_uint2(pack_bf16x2(p.x, p.y), pack_bf16x2(p.z, p.w));
  }
  for (long long i = (nvec << 2) + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p = master[i], m = exp_avg[i], v = exp_avg_sq[i];
    update(__bfloat162float(grad[i]), p, m, v);
    master[i] = p;
    exp_avg[i] = m;
    exp_avg_sq[i] = v;
    param_out[i] = __float2bfloat16_rn(p);
  }
}

// A wait that nothing satisfies: used to exercise the bounded-wait path on one GPU.
__global__ void wait_probe_kernel(const unsigned int* flag, unsigned long long limit_ns, uint32_t* status) {
  const uint64_t t0 = globaltimer_ns();
  while (*reinterpret_cast<const volatile unsigned int*>(flag) == 0u) {
    if (globaltimer_ns() - t0 > limit_ns) {
      record_status(status, STATUS_TIMEOUT_TEST_FLAG, 0u);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace

extern "C" {

int gfs_ce_fwd(const void* logits, const void* target, void* stats, void* lse, void* loss, int M, int Vp, long ld,
               int v0, int single_rank, void* stream) {
  if ((Vp & 7) || (ld & 7)) return -1;
  if (M == 0) return 0;
  ce_fwd_kernel<<<M, CE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), static_cast<const long long*>(target), static_cast<float*>(stats),
      static_cast<float*>(lse), static_cast<float*>(loss), Vp, ld, v0, single_rank);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_ce_from_partials(const void* partials, const void* logits, const void* target, void* stats, void* lse,
                         void* loss, int parts, int M, int Vp, long ld, int v0, int single_rank, void* stream) {
  if (M == 0) return 0;
  ce_from_partials_kernel<<<(M + 31) / 32, 32 * CE_PW, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float2*>(partials), static_cast<const __nv_bfloat16*>(logits),
      static_cast<const long long*>(target), static_cast<float*>(stats), static_cast<float*>(lse),
      static_cast<float*>(loss), parts, M, Vp, ld, v0, single_rank);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_ce_combine(const void* stats_all, void* lse, void* loss, int M, int world, void* stream) {
  if (M == 0) return 0;
  ce_combine_kernel<<<(M + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(stats_all), static_cast<float*>(lse), static_cast<float*>(loss), M, world);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_ce_bwd(void* logits, const void* lse, const void* target, const void* grad_rows, int M, int Vp, long ld,
               int v0, void* stream) {
  if ((Vp & 7) || (ld & 7)) return -1;
  if (M == 0 || Vp == 0) return 0;
  const dim3 grid(((Vp >> 3) + 255) / 256, std::min((M + 3) / 4, 1024));
  ce_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), static_cast<const float*>(lse), static_cast<const long long*>(target),
      static_cast<const float*>(grad_rows), M, Vp, ld, v0);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// scratch: at least gfs_sumsq_scratch_bytes() bytes, zero-initialised once by the caller.
int gfs_sumsq_scratch_bytes() { return (SUMSQ_MAX_BLOCKS + 4) * 4; }

int gfs_sumsq_bf16(const void* x, long long n, void* out, void* scratch, void* stream) {
  const long long nvec = n >> 3;
  long long blocks = (nvec + SUMSQ_THREADS - 1) / SUMSQ_THREADS;
  blocks = std::max<long long>(1, std::min<long long>(blocks, std::min(SUMSQ_MAX_BLOCKS, gfs_host::sm_count() * 4)));
  sumsq_bf16_kernel<<<static_cast<int>(blocks), SUMSQ_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), n, static_cast<float*>(out), static_cast<float*>(scratch));
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// sumsq: device scalar with the squared norm of the (unscaled) gradient over all shards, or null
// to skip clipping. norm_out (optional) receives the scaled norm. step_dev (optional): device
// float holding the step count t; when set the kernel derives the bias corrections from it
// (beta1, beta2 as doubles) and ignores bias_corr1 / bias_corr2_sqrt.
int gfs_adamw_step(const void* grad, void* master, void* exp_avg, void* exp_avg_sq, void* param_out, long long n,
                   const void* sumsq, void* norm_out, float lr, double beta1, double beta2, float eps,
                   float weight_decay, float bias_corr1, float bias_corr2_sqrt, float clip, float grad_scale,
                   const void* step_dev, void* stream) {
  if (n == 0) return 0;
  AdamArgs a{lr, static_cast<float>(beta1), static_cast<float>(beta2), eps, weight_decay, bias_corr1,
             bias_corr2_sqrt, clip, grad_scale, static_cast<const float*>(step_dev), beta1, beta2};
  const long long blocks =
      std::max<long long>(1, std::min<long long>((n / 4 + 255) / 256, static_cast<long long>(gfs_host::sm_count()) * 16));
  adamw_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(grad), static_cast<float*>(master), static_cast<float*>(exp_avg),
      static_cast<float*>(exp_avg_sq), static_cast<__nv_bfloat16*>(param_out), n, static_cast<const float*>(sumsq),
      static_cast<float*>(norm_out), a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Launches a kernel that waits (at most limit_ns) for *flag != 0. If the flag is never set the
// kernel records STATUS_TIMEOUT_TEST_FLAG and returns; the context stays usable.
int gfs_wait_probe(const void* flag, long long limit_ns, void* stream) {
  if (limit_ns > 2000000000ll) limit_ns = 2000000000ll;
  wait_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned int*>(flag),
                                                                   static_cast<unsigned long long>(limit_ns),
                                                                   gfs_host::status_words());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
