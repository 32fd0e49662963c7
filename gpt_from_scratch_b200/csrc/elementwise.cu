// Memory-bound kernels of the training step: RMSNorm fwd/bwd, rotary embedding,
// SwiGLU fwd/bwd, embedding lookup fwd/bwd. Each replaces a chain of ATen kernels of
// the reference with one pass over the data (16-byte vector accesses, fp32 math).
//
// Reference counterparts: core/normalization.py:13-25 (RMSNorm), core/rope_triton.py:74-141
// (RoPE), core/mlp.py:25-28 (SwiGLU), core/tensor_parallel/layers.py:117-134 (embedding).
#include <algorithm>

#include "common.cuh"

using namespace gfs;

namespace {

constexpr int NORM_WARPS = 4;

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
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---------------------------------------------------------------------------
// RMSNorm forward: y = bf16(x * rstd) * w, rstd = rsqrt(mean(x^2) + eps). One warp per row.
// ---------------------------------------------------------------------------
// NORM_MAXV = vectors of 8 bf16 cached per lane (covers H <= 256 * NORM_MAXV without a second
// read); a template parameter so that small hidden sizes do not pay for 64 cache registers.
template <int NORM_MAXV>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, int H, float eps) {
  pdl_wait();       // launched programmatically: the preceding kernel's output is complete from here on
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = H >> 3;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * H;
  uint4 cache[NORM_MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      cache[i] = *reinterpret_cast<const uint4*>(xr + 8 * v);
      const float2 a = unpack_bf16x2(cache[i].x), b = unpack_bf16x2(cache[i].y), c = unpack_bf16x2(cache[i].z),
                   d = unpack_bf16x2(cache[i].w);
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
    }
  }
  for (int v = lane + 32 * NORM_MAXV; v < nvec; v += 32) {
    float f[8];
    load8(xr + 8 * v, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float f[8], g[8];
      const float2 a = unpack_bf16x2(cache[i].x), b = unpack_bf16x2(cache[i].y), c = unpack_bf16x2(cache[i].z),
                   d = unpack_bf16x2(cache[i].w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
      load8(w + 8 * v, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = round_bf16(f[e] * rstd) * g[e];
      store8(yr + 8 * v, f);
    }
  }
  for (int v = lane + 32 * NORM_MAXV; v < nvec; v += 32) {
    float f[8], g[8];
    load8(xr + 8 * v, f);
    load8(w + 8 * v, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = round_bf16(f[e] * rstd) * g[e];
    store8(yr + 8 * v, f);
  }
}

// ---------------------------------------------------------------------------
// RMSNorm backward. Each CTA owns a contiguous block of rows; every warp keeps the
// weight-gradient partial of the rows it handled in its own shared-memory row, so dw
// needs no atomics: per-CTA partials [gridDim.x, H] are summed by a second kernel.
//   g = dy * w;  dx = rstd * g - x * rstd^3 * mean(g * x)  (+ dres);  dw += dy * bf16(x * rstd)
// ---------------------------------------------------------------------------
constexpr int NB_WARPS = 8;

// Register path (H <= 256 * NV): every lane keeps the row values it needs for the second
// pass and its dw partial sums in registers; shared memory is only used once at the end.
template <int NV>
__global__ void __launch_bounds__(NB_WARPS * 32, NV <= 4 ? 2 : 1)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, int rows, int H, int rows_per_cta) {
  extern __shared__ float red[];  // [warps][H]
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int nvec = H >> 3;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(rows, r0 + rows_per_cta);
  float wv[NV][8];
  float dwacc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dwacc[i][e] = 0.f;
      wv[i][e] = 0.f;
    }
    if (v < nvec) load8(w + 8 * v, wv[i]);
  }
  for (int row = r0 + warp; row < r1; row += nwarps) {
    const __nv_bfloat16* dyr = dy + static_cast<size_t>(row) * H;
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    const float rs = rstd[row];
    uint4 cdy[NV], cx[NV], cres[NV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        cdy[i] = *reinterpret_cast<const uint4*>(dyr + 8 * v);
        cx[i] = *reinterpret_cast<const uint4*>(xr + 8 * v);
        if (dres != nullptr) cres[i] = *reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * H + 8 * v);
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        const float2 a0 = unpack_bf16x2(cdy[i].x), a1 = unpack_bf16x2(cdy[i].y), a2 = unpack_bf16x2(cdy[i].z),
                     a3 = unpack_bf16x2(cdy[i].w);
        const float2 b0 = unpack_bf16x2(cx[i].x), b1 = unpack_bf16x2(cx[i].y), b2 = unpack_bf16x2(cx[i].z),
                     b3 = unpack_bf16x2(cx[i].w);
        dot += a0.x * wv[i][0] * b0.x + a0.y * wv[i][1] * b0.y + a1.x * wv[i][2] * b1.x + a1.y * wv[i][3] * b1.y +
               a2.x * wv[i][4] * b2.x + a2.y * wv[i][5] * b2.y + a3.x * wv[i][6] * b3.x + a3.y * wv[i][7] * b3.y;
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * rs * rs * rs / static_cast<float>(H);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float a[8], b[8], o[8];
        const float2 a0 = unpack_bf16x2(cdy[i].x), a1 = unpack_bf16x2(cdy[i].y), a2 = unpack_bf16x2(cdy[i].z),
                     a3 = unpack_bf16x2(cdy[i].w);
        const float2 b0 = unpack_bf16x2(cx[i].x), b1 = unpack_bf16x2(cx[i].y), b2 = unpack_bf16x2(cx[i].z),
                     b3 = unpack_bf16x2(cx[i].w);
        a[0] = a0.x; a[1] = a0.y; a[2] = a1.x; a[3] = a1.y; a[4] = a2.x; a[5] = a2.y; a[6] = a3.x; a[7] = a3.y;
        b[0] = b0.x; b[1] = b0.y; b[2] = b1.x; b[3] = b1.y; b[4] = b2.x; b[5] = b2.y; b[6] = b3.x; b[7] = b3.y;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o[e] = rs * a[e] * wv[i][e] - b[e] * coef;
          dwacc[i][e] += a[e] * round_bf16(b[e] * rs);
        }
        if (dres != nullptr) {
          const float2 d0 = unpack_bf16x2(cres[i].x), d1 = unpack_bf16x2(cres[i].y), d2 = unpack_bf16x2(cres[i].z),
                       d3 = unpack_bf16x2(cres[i].w);
          o[0] += d0.x; o[1] += d0.y; o[2] += d1.x; o[3] += d1.y; o[4] += d2.x; o[5] += d2.y; o[6] += d3.x; o[7] += d3.y;
        }
        store8(dx + static_cast<size_t>(row) * H + 8 * v, o);
      }
    }
  }
  float* my_red = red + static_cast<size_t>(warp) * H;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) my_red[8 * v + e] = dwacc[i][e];
    }
  }
  __syncthreads();
  float* outp = dw_partial + static_cast<size_t>(blockIdx.x) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float s = 0.f;
    for (int wv2 = 0; wv2 < nwarps; ++wv2) s += red[static_cast<size_t>(wv2) * H + i];
    outp[i] = s;
  }
}

// Generic path (any H that is a multiple of 8): partial sums live in shared memory.
__global__ void __launch_bounds__(NB_WARPS * 32)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int H, int rows_per_cta) {
  extern __shared__ float red[];  // [warps][H]
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int nvec = H >> 3;
  const int r0 = blockIdx.x * rows_per_cta;
  const int r1 = min(rows, r0 + rows_per_cta);
  float* my_red = red + static_cast<size_t>(warp) * H;
  for (int i = lane; i < H; i += 32) my_red[i] = 0.f;
  __syncwarp();

  for (int row = r0 + warp; row < r1; row += nwarps) {
    const __nv_bfloat16* dyr = dy + static_cast<size_t>(row) * H;
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    __nv_bfloat16* dxr = dx + static_cast<size_t>(row) * H;
    const float rs = rstd[row];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float a[8], b[8], c[8];
      load8(dyr + 8 * v, a);
      load8(xr + 8 * v, b);
      load8(w + 8 * v, c);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += a[e] * c[e] * b[e];
    }
    dot = warp_sum(dot);
    const float coef = dot * rs * rs * rs / static_cast<float>(H);
    for (int v = lane; v < nvec; v += 32) {
      float a[8], b[8], c[8], o[8];
      load8(dyr + 8 * v, a);
      load8(xr + 8 * v, b);
      load8(w + 8 * v, c);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rs * a[e] * c[e] - b[e] * coef;
      if (dres != nullptr) {
        float d[8];
        load8(dres + static_cast<size_t>(row) * H + 8 * v, d);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += d[e];
      }
      store8(dxr + 8 * v, o);
      float* acc = my_red + 8 * v;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += a[e] * round_bf16(b[e] * rs);
    }
  }
  __syncthreads();
  float* outp = dw_partial + static_cast<size_t>(blockIdx.x) * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float s = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) s += red[static_cast<size_t>(wv) * H + i];
    outp[i] = s;
  }
}

// blockDim = (32, 32): 32 columns per block, the partial rows are split over 32 thread rows and
// combined through shared memory in a fixed order (deterministic).
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int parts,
                                         int H, int accumulate) {
  __shared__ float sm[32][33];
  const int i = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (i < H) {
    for (int p = threadIdx.y; p < parts; p += 32) s += partial[static_cast<size_t>(p) * H + i];
  }
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < H) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += sm[y][threadIdx.x];
    if (accumulate) t += __bfloat162float(dw[i]);
    dw[i] = __float2bfloat16_rn(t);
  }
}

// The same reduction for several RMSNorm layers in one launch (blockIdx.y = layer): the
// per-layer reductions are tiny, so a backward pass parks them and runs them together.
constexpr int DW_MULTI_MAX = 32;
struct DwReduceBatch {
  const float* partial[DW_MULTI_MAX];
  __nv_bfloat16* dw[DW_MULTI_MAX];
  int parts[DW_MULTI_MAX];
  int accumulate[DW_MULTI_MAX];
};

__global__ void rmsnorm_dw_reduce_multi_kernel(const __grid_constant__ DwReduceBatch b, int H) {
  __shared__ float sm[32][33];
  const int l = blockIdx.y;
  const float* __restrict__ partial = b.partial[l];
  __nv_bfloat16* __restrict__ dw = b.dw[l];
  const int parts = b.parts[l];
  const int i = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (i < H) {
    for (int p = threadIdx.y; p < parts; p += 32) s += partial[static_cast<size_t>(p) * H + i];
  }
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < H) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += sm[y][threadIdx.x];
    if (b.accumulate[l]) t += __bfloat162float(dw[i]);
    dw[i] = __float2bfloat16_rn(t);
  }
}

// ---------------------------------------------------------------------------
// Rotary embedding, interleaved pairs, in place on `parts` consecutive [nh*D] blocks
// of every token (parts = 2: the q and k thirds of a [S,B,3,nh,D] buffer).
//   x'[2i] = x[2i] cos - x[2i+1] sin ; x'[2i+1] = x[2i] sin + x[2i+1] cos ; backward: sin -> -sin
// ---------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cosb,
                            const float* __restrict__ sinb, int S, int B, int nhD, int D, int parts,
                            long token_stride, int backward, int s_offset) {
  const int vec_per_token = (parts * nhD) >> 3;
  const size_t total = static_cast<size_t>(S) * B * vec_per_token;
  for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < total;
       v += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t token = v / vec_per_token;
    const int e0 = static_cast<int>(v % vec_per_token) << 3;
    const int s = static_cast<int>(token / B) + s_offset;
    const int d = e0 % D;
    __nv_bfloat16* p = x + token * token_stride + e0;
    float f[8];
    load8(p, f);
    const float4 c = *reinterpret_cast<const float4*>(cosb + static_cast<size_t>(s) * (D >> 1) + (d >> 1));
    float4 sn = *reinterpret_cast<const float4*>(sinb + static_cast<size_t>(s) * (D >> 1) + (d >> 1));
    if (backward) {
      sn.x = -sn.x; sn.y = -sn.y; sn.z = -sn.z; sn.w = -sn.w;
    }
    float o[8];
    o[0] = f[0] * c.x - f[1] * sn.x; o[1] = f[0] * sn.x + f[1] * c.x;
    o[2] = f[2] * c.y - f[3] * sn.y; o[3] = f[2] * sn.y + f[3] * c.y;
    o[4] = f[4] * c.z - f[5] * sn.z; o[5] = f[4] * sn.z + f[5] * c.z;
    o[6] = f[6] * c.w - f[7] * sn.w; o[7] = f[6] * sn.w + f[7] * c.w;
    store8(p, o);
  }
}

// ---------------------------------------------------------------------------
// Dropout fused with the residual add (the reference's `residual + dropout(x)`,
// core/transformer_layer.py:97,103). Counter-based generator: one 64-bit mix of
// (seed, vector index) yields the eight 8-bit thresholds of a vector of 8 elements, so
// the keep probability is quantised to 1/256 and no mask tensor exists.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

__global__ void dropout_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                        __nv_bfloat16* __restrict__ out, long long nvec, float p,
                                        unsigned long long seed, int backward) {
  const unsigned int drop_below = static_cast<unsigned int>(p * 256.f + 0.5f);  // byte < drop_below -> dropped
  const float scale = 256.f / static_cast<float>(256u - drop_below);           // 1 / (realised keep probability)
  for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned long long bits = mix64(seed ^ (static_cast<unsigned long long>(v) * 0xd1342543de82ef95ull));
    float f[8], r[8], o[8];
    load8(x + 8 * v, f);
    if (!backward && residual != nullptr) load8(residual + 8 * v, r);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const bool keep = ((bits >> (8 * e)) & 0xffull) >= drop_below;
      const float d = keep ? f[e] * scale : 0.f;
      o[e] = (!backward && residual != nullptr) ? r[e] + round_bf16(d) : d;
    }
    store8(out + 8 * v, o);
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on a [M, 2I] buffer whose first I columns are the gate and last I the up half.
// ---------------------------------------------------------------------------
// Grid: x covers the 8-column vectors of a row, y strides over rows (no integer divisions).
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int M, int I) {
  const int vec_per_row = I >> 3;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vec_per_row) return;
  const int c = v << 3;
  for (int row = blockIdx.y; row < M; row += gridDim.y) {
    const __nv_bfloat16* base = gu + static_cast<size_t>(row) * 2 * I;
    float g[8], u[8], o[8];
    load8(base + c, g);
    load8(base + I + c, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = __fdividef(1.f, 1.f + __expf(-g[e]));
      // silu rounded to bf16 before the product, as two separate bf16 ops would do
      o[e] = round_bf16(g[e] * sg) * u[e];
    }
    store8(act + static_cast<size_t>(row) * I + c, o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, int M, int I) {
  const int vec_per_row = I >> 3;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= vec_per_row) return;
  const int c = v << 3;
  for (int row = blockIdx.y; row < M; row += gridDim.y) {
    const size_t rb = static_cast<size_t>(row) * 2 * I;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + rb + c, g);
    load8(gu + rb + I + c, u);
    load8(dact + static_cast<size_t>(row) * I + c, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = __fdividef(1.f, 1.f + __expf(-g[e]));
      const float silu = g[e] * sg;
      dg[e] = d[e] * u[e] * sg * (1.f + g[e] * (1.f - sg));
      du[e] = d[e] * silu;
    }
    store8(dgu + rb + c, dg);
    store8(dgu + rb + I + c, du);
  }
}

// ---------------------------------------------------------------------------
// Embedding forward: out[s - s0, b, :] = W[id - v0] if v0 <= id < v1 else 0, ids are [B, S].
// One warp per output row.
// ---------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ W,
                                     __nv_bfloat16* __restrict__ out, int B, int S, int H, int v0, int v1, int s0,
                                     int s_count) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= s_count * B) return;
  const int s = s0 + r / B;
  const int b = r % B;
  const long long id = ids[static_cast<size_t>(b) * S + s];
  __nv_bfloat16* o = out + static_cast<size_t>(r) * H;
  const int nvec = H >> 3;
  if (id >= v0 && id < v1) {
    const __nv_bfloat16* src = W + static_cast<size_t>(id - v0) * H;
    for (int v = lane; v < nvec; v += 32)
      *reinterpret_cast<uint4*>(o + 8 * v) = *reinterpret_cast<const uint4*>(src + 8 * v);
  } else {
    for (int v = lane; v < nvec; v += 32) *reinterpret_cast<uint4*>(o + 8 * v) = make_uint4(0, 0, 0, 0);
  }
}

// Embedding backward over token ids sorted ascending (perm gives each sorted position's
// row in dout). A warp owns one run of equal ids and sums its rows in sorted order,
// so the result is deterministic; dW rows are accumulated (bf16, fp32 sum).
__global__ void embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ perm,
                                     const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dW, int n,
                                     int H, int v0, int v1) {
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= n) return;
  const long long id = sorted_ids[p];
  if (id < v0 || id >= v1) return;
  if (p > 0 && sorted_ids[p - 1] == id) return;  // not the start of a run
  int q_end = p + 1;
  while (q_end < n && sorted_ids[q_end] == id) ++q_end;
  __nv_bfloat16* dst = dW + static_cast<size_t>(id - v0) * H;
  const int nvec = H >> 3;
  for (int v = lane; v < nvec; v += 32) {
    float acc[8];
    load8(dst + 8 * v, acc);
    for (int q = p; q < q_end; ++q) {
      float f[8];
      load8(dout + static_cast<size_t>(perm[q]) * H + 8 * v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    store8(dst + 8 * v, acc);
  }
}

// Embedding backward without a library sort: the token ids of one micro-batch (n <= 32768) are
// sorted by ONE CTA in shared memory. Key = (local vocabulary row << shift) | dout row index, so
// keys are unique and ascending order is "by row, then by position" - the order a stable sort
// gives, hence the same bitwise result as summing in sorted order. Ids owned by other ranks get
// the all-ones key and end up behind the valid ones. Bitonic network on npow2 keys.
constexpr int SORT_THREADS = 1024;
__global__ void __launch_bounds__(SORT_THREADS)
embedding_sort_kernel(const long long* __restrict__ ids_bs, uint32_t* __restrict__ keys_out, int n, int npow2,
                      int shift, int B, int S, int v0, int v1) {
  extern __shared__ uint32_t sk[];
  for (int i = threadIdx.x; i < npow2; i += SORT_THREADS) {
    uint32_t key = 0xFFFFFFFFu;
    if (i < n) {
      const long long id = ids_bs[static_cast<size_t>(i % B) * S + i / B];   // dout row i = (s, b) = (i / B, i % B)
      if (id >= v0 && id < v1) key = (static_cast<uint32_t>(id - v0) << shift) | static_cast<uint32_t>(i);
    }
    sk[i] = key;
  }
  __syncthreads();
  for (int k = 2; k <= npow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int c = threadIdx.x; c < (npow2 >> 1); c += SORT_THREADS) {
        const int a = ((c & ~(j - 1)) << 1) | (c & (j - 1));
        const int b = a | j;
        const uint32_t x = sk[a], y = sk[b];
        const bool ascending = (a & k) == 0;
        if ((x > y) == ascending) {
          sk[a] = y;
          sk[b] = x;
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < n; i += SORT_THREADS) keys_out[i] = sk[i];
}

// Segmented sum over the sorted keys: a warp owns one run of equal vocabulary rows and adds its
// dout rows in key order (deterministic); dW rows are accumulated (bf16, fp32 sum).
__global__ void embedding_bwd_keys_kernel(const uint32_t* __restrict__ keys, const __nv_bfloat16* __restrict__ dout,
                                          __nv_bfloat16* __restrict__ dW, int n, int H, int shift) {
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= n) return;
  const uint32_t key = keys[p];
  if (key == 0xFFFFFFFFu) return;
  const uint32_t row = key >> shift;
  if (p > 0 && (keys[p - 1] >> shift) == row) return;  // not the start of a run
  const uint32_t mask = (1u << shift) - 1u;
  int q_end = p + 1;
  while (q_end < n && keys[q_end] != 0xFFFFFFFFu && (keys[q_end] >> shift) == row) ++q_end;
  __nv_bfloat16* dst = dW + static_cast<size_t>(row) * H;
  const int nvec = H >> 3;
  for (int v = lane; v < nvec; v += 32) {
    float acc[8];
    load8(dst + 8 * v, acc);
    for (int q = p; q < q_end; ++q) {
      float f[8];
      load8(dout + static_cast<size_t>(keys[q] & mask) * H + 8 * v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    store8(dst + 8 * v, acc);
  }
}

inline int grid_for(size_t work_items, int threads, int max_blocks_per_sm = 16) {
  const size_t blocks = (work_items + threads - 1) / threads;
  const size_t cap = static_cast<size_t>(gfs_host::sm_count()) * max_blocks_per_sm;
  return static_cast<int>(std::max<size_t>(1, std::min(blocks, cap)));
}

}  // namespace

extern "C" {

int gfs_rmsnorm_fwd(const void* x, const void* w, void* y, void* rstd, int rows, int H, float eps, void* stream) {
  if (H & 7) return -1;
  if (rows == 0) return 0;
  const int blocks = (rows + NORM_WARPS - 1) / NORM_WARPS;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  float* rp = static_cast<float*>(rstd);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(blocks), block(NORM_WARPS * 32);
  if (H <= 1024) gfs_host::launch_pdl(rmsnorm_fwd_kernel<4>, grid, block, 0, st, xp, wp, yp, rp, rows, H, eps);
  else if (H <= 2048) gfs_host::launch_pdl(rmsnorm_fwd_kernel<8>, grid, block, 0, st, xp, wp, yp, rp, rows, H, eps);
  else gfs_host::launch_pdl(rmsnorm_fwd_kernel<16>, grid, block, 0, st, xp, wp, yp, rp, rows, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Number of fp32 elements the backward needs in `partial`: parts * H with parts from this call.
int gfs_rmsnorm_bwd_parts(int rows) {
  const int sms = gfs_host::sm_count();
  const int want = sms * 2;   // one resident wave (two CTAs per SM): 39 -> 34 us at 16384 x 768
  const int rows_per_cta = std::max(NB_WARPS, (rows + want - 1) / want);
  return (rows + rows_per_cta - 1) / rows_per_cta;
}

// dx = rmsnorm backward (+ dres); dw (bf16 [H]) written or accumulated. partial: fp32 scratch [parts*H].
int gfs_rmsnorm_bwd(const void* dy, const void* x, const void* w, const void* rstd, const void* dres, void* dx,
                    void* dw, void* partial, int rows, int H, int accumulate_dw, void* stream_) {
  if (H & 7) return -1;
  if (rows == 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int parts = gfs_rmsnorm_bwd_parts(rows);
  const int rows_per_cta = (rows + parts - 1) / parts;
  int warps = NB_WARPS;
  while (warps > 1 && static_cast<size_t>(warps) * H * sizeof(float) > 200 * 1024) warps >>= 1;
  const size_t smem = static_cast<size_t>(warps) * H * sizeof(float);
  if (smem > 200 * 1024) return -1;
  const __nv_bfloat16* a_dy = static_cast<const __nv_bfloat16*>(dy);
  const __nv_bfloat16* a_x = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* a_w = static_cast<const __nv_bfloat16*>(w);
  const float* a_rstd = static_cast<const float*>(rstd);
  const __nv_bfloat16* a_res = static_cast<const __nv_bfloat16*>(dres);
  __nv_bfloat16* a_dx = static_cast<__nv_bfloat16*>(dx);
  float* a_part = static_cast<float*>(partial);
  auto ensure_smem = [&](auto kern, int& done) -> int {
    if (smem > 48 * 1024 && done < static_cast<int>(smem)) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return -10;
      done = 200 * 1024;
    }
    return 0;
  };
  static int set_gen = 0, set_r4 = 0, set_r8 = 0;
  if (H <= 1024) {
    if (ensure_smem(rmsnorm_bwd_reg_kernel<4>, set_r4)) return -10;
    gfs_host::launch_pdl(rmsnorm_bwd_reg_kernel<4>, dim3(parts), dim3(warps * 32), smem, stream, a_dy, a_x, a_w, a_rstd,
                         a_res, a_dx, a_part, rows, H, rows_per_cta);
  } else if (H <= 2048) {
    if (ensure_smem(rmsnorm_bwd_reg_kernel<8>, set_r8)) return -10;
    gfs_host::launch_pdl(rmsnorm_bwd_reg_kernel<8>, dim3(parts), dim3(warps * 32), smem, stream, a_dy, a_x, a_w, a_rstd,
                         a_res, a_dx, a_part, rows, H, rows_per_cta);
  } else {
    if (ensure_smem(rmsnorm_bwd_kernel, set_gen)) return -10;
    gfs_host::launch_pdl(rmsnorm_bwd_kernel, dim3(parts), dim3(warps * 32), smem, stream, a_dy, a_x, a_w, a_rstd, a_res,
                         a_dx, a_part, rows, H, rows_per_cta);
  }
  if (cudaGetLastError() != cudaSuccess) return -11;
  if (dw == nullptr) return 0;   // the caller reduces `partial` later (gfs_rmsnorm_dw_reduce_multi)
  rmsnorm_dw_reduce_kernel<<<(H + 31) / 32, dim3(32, 32), 0, stream>>>(static_cast<const float*>(partial),
                                                              static_cast<__nv_bfloat16*>(dw), parts, H,
                                                              accumulate_dw);
  return cudaGetLastError() == cudaSuccess ? 0 : -12;
}

// Weight-gradient reductions of n RMSNorm layers (n <= 32) that ran gfs_rmsnorm_bwd with dw == null:
// dw_l (bf16 [H]) = (or +=) column sums of partial_l (fp32 [parts_l, H]).
int gfs_rmsnorm_dw_reduce_multi(int n, const unsigned long long* partial, const unsigned long long* dw,
                                const int* parts, const int* accumulate, int H, void* stream) {
  if (n <= 0) return 0;
  if (n > DW_MULTI_MAX) return -1;
  DwReduceBatch b{};
  for (int i = 0; i < n; ++i) {
    b.partial[i] = reinterpret_cast<const float*>(partial[i]);
    b.dw[i] = reinterpret_cast<__nv_bfloat16*>(dw[i]);
    b.parts[i] = parts[i];
    b.accumulate[i] = accumulate[i];
  }
  rmsnorm_dw_reduce_multi_kernel<<<dim3((H + 31) / 32, n), dim3(32, 32), 0, static_cast<cudaStream_t>(stream)>>>(b, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_rope(void* x, const void* cosb, const void* sinb, int S, int B, int nh, int D, int parts, long token_stride,
             int backward, int s_offset, void* stream) {
  if ((D & 7) || (token_stride & 7)) return -1;
  const size_t total = static_cast<size_t>(S) * B * ((static_cast<size_t>(parts) * nh * D) >> 3);
  if (total == 0) return 0;
  rope_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const float*>(cosb), static_cast<const float*>(sinb), S, B, nh * D,
      D, parts, token_stride, backward, s_offset);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// out = residual + dropout(x, p) (forward) or dx = dy * keep / (1 - p) (backward, mode 1). The keep
// mask is a pure function of (seed, element index), so the backward regenerates it instead of
// storing it; n is a multiple of 8.
int gfs_dropout_residual(const void* x, const void* residual, void* out, long long n, float p, unsigned long long seed,
                         int backward, void* stream) {
  if (n & 7) return -1;
  if (n == 0) return 0;
  if (!(p >= 0.f) || p >= 1.f) return -1;
  const long long nvec = n >> 3;
  const int blocks = static_cast<int>(std::min<long long>((nvec + 255) / 256, static_cast<long long>(gfs_host::sm_count()) * 16));
  dropout_residual_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(out), nvec, p, seed, backward);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_swiglu_fwd(const void* gu, void* act, int M, int I, void* stream) {
  if (I & 7) return -1;
  if (M == 0 || I == 0) return 0;
  const dim3 grid(((I >> 3) + 127) / 128, std::min(M, 32768));
  swiglu_fwd_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(act), M, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_swiglu_bwd(const void* dact, const void* gu, void* dgu, int M, int I, void* stream) {
  if (I & 7) return -1;
  if (M == 0 || I == 0) return 0;
  const dim3 grid(((I >> 3) + 127) / 128, std::min(M, 32768));
  swiglu_bwd_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dact), static_cast<const __nv_bfloat16*>(gu),
      static_cast<__nv_bfloat16*>(dgu), M, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_embedding_fwd(const void* ids, const void* W, void* out, int B, int S, int H, int v0, int v1, int s0,
                      int s_count, void* stream) {
  if (H & 7) return -1;
  const int rows = s_count * B;
  if (rows == 0) return 0;
  const int warps = 8;
  embedding_fwd_kernel<<<(rows + warps - 1) / warps, warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(W), static_cast<__nv_bfloat16*>(out), B, S,
      H, v0, v1, s0, s_count);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_embedding_bwd(const void* sorted_ids, const void* perm, const void* dout, void* dW, int n, int H, int v0,
                      int v1, void* stream) {
  if (H & 7) return -1;
  if (n == 0) return 0;
  const int warps = 8;
  embedding_bwd_kernel<<<(n + warps - 1) / warps, warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(sorted_ids), static_cast<const long long*>(perm),
      static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dW), n, H, v0, v1);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Embedding backward with the in-library sort, in two calls so that the sort (one CTA, tens of
// microseconds, needs only the token ids) can run on a side stream during the forward pass:
//   gfs_embedding_sort_keys  ids [B, S] (int64) -> keys [S * B] uint32, sorted; returns the key
//                            shift (> 0), or -20 when the problem does not fit the single-CTA sort
//                            (n > 32768 or the key does not fit 32 bits: the caller then sorts
//                            elsewhere and uses gfs_embedding_bwd)
//   gfs_embedding_bwd_keys   dW [v1 - v0, H] += segmented sum of dout [S, B, H] in key order
int gfs_embedding_sort_keys(const void* ids_bs, void* keys, int B, int S, int v0, int v1, void* stream_) {
  const long long n64 = static_cast<long long>(B) * S;
  if (n64 <= 0) return -1;
  if (n64 > 32768) return -20;
  const int n = static_cast<int>(n64);
  int npow2 = 2, shift = 1;
  while (npow2 < n) { npow2 <<= 1; ++shift; }
  if ((static_cast<unsigned long long>(v1 - v0) << shift) >= 0xFFFFFFFFull) return -20;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(embedding_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4) !=
        cudaSuccess)
      return -10;
    attr_set = true;
  }
  embedding_sort_kernel<<<1, SORT_THREADS, npow2 * sizeof(uint32_t), stream>>>(
      static_cast<const long long*>(ids_bs), static_cast<uint32_t*>(keys), n, npow2, shift, B, S, v0, v1);
  return cudaGetLastError() == cudaSuccess ? shift : -11;
}

int gfs_embedding_bwd_keys(const void* keys, const void* dout, void* dW, int n, int H, int shift, void* stream_) {
  if ((H & 7) || shift <= 0 || shift > 31) return -1;
  if (n == 0) return 0;
  const int warps = 8;
  embedding_bwd_keys_kernel<<<(n + warps - 1) / warps, warps * 32, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint32_t*>(keys), static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dW), n, H,
      shift);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
