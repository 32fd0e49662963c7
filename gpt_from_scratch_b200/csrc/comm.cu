// Collectives done by our own kernels over peer memory (NVLink / NVSwitch), fused with the
// elementwise work around them. Buffers are symmetric allocations: every rank passes the
// table of all ranks' pointers. Signalling uses monotonically growing uint32 counters in
// the destination's memory (flags[dst][src]) and host-tracked cumulative targets; every
// wait is bounded and reports STATUS_TIMEOUT_PEER_FLAG instead of hanging.
//
//   gfs_symm_barrier        cross-rank barrier (used sparingly, e.g. once per optimizer step)
//   gfs_allgather           push-style all-gather of a row block
//   gfs_embedding_scatter   vocab-parallel embedding lookup whose rows are written straight
//                           into the sequence-shard owner's output (lookup + reduce-scatter)
//   gfs_ce_exchange         vocab-parallel cross entropy: exchange of (max, sum-exp, target
//                           logit) and the combine into lse / loss, replacing two all-reduces
//   gfs_dp_push_grads       data-parallel gradient reduce-scatter, part 1: per-bucket push of the
//                           peers' slices into their staging buffers (overlaps the backward pass)
//   gfs_dp_sum_norm         part 2: sum of the staged contributions + squared-norm partial
//   gfs_dp_adam_gather      global-norm clip + AdamW on the fp32 shard + bf16 parameter
//                           all-gather by peer stores
//
// Reference counterparts: the NCCL calls in core/tensor_parallel/mappings.py:22,35,
// core/tensor_parallel/loss.py:15,45, core/tensor_parallel/layers.py:134 and
// core/optimizer.py:81,95,101.
#include <algorithm>

#include "common.cuh"

using namespace gfs;

namespace {

constexpr int MAX_PEERS = 8;

struct PeerTable {
  void* buf[MAX_PEERS];
  uint32_t* flags[MAX_PEERS];
};

// Every CTA signals each destination once, then waits until each source has signalled
// `target` times in total. Called by all threads of the CTA after their stores.
__device__ __forceinline__ void cta_signal_all_and_wait(const PeerTable& t, int world, int rank, int slot0,
                                                        uint32_t target, unsigned long long wait_ns,
                                                        uint32_t* status) {
  __syncthreads();   // orders every thread's stores before the releases below (which are cumulative)
  if (threadIdx.x < world) red_release_sys_add_u32(t.flags[threadIdx.x] + slot0 + rank, 1u);
  if (threadIdx.x < world)
    wait_flag_reached(t.flags[rank] + slot0 + threadIdx.x, target, wait_ns, status,
                      0xC0000000u | (slot0 << 8) | (threadIdx.x << 4) | rank);
  __syncthreads();
}

// ---------------------------------------------------------------------------
__global__ void symm_barrier_kernel(PeerTable t, int world, int rank, int slot0, uint32_t target,
                                    unsigned long long wait_ns, uint32_t* status) {
  cta_signal_all_and_wait(t, world, rank, slot0, target, wait_ns, status);
}

// ---------------------------------------------------------------------------
// All-gather: src [rows, cols] (pitch ld) -> rows [rank*rows, (rank+1)*rows) of every rank's buffer.
__global__ void allgather_kernel(PeerTable t, const __nv_bfloat16* __restrict__ src, int rows, int cols, int ld,
                                 int world, int rank, int slot0, uint32_t target, unsigned long long wait_ns,
                                 uint32_t* status) {
  const int vpr = cols >> 3;
  const size_t total = static_cast<size_t>(rows) * vpr;
  for (int i = 0; i < world; ++i) {
    const int peer = (rank + i) % world;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(t.buf[peer]) + static_cast<size_t>(rank) * rows * cols;
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < total;
         v += static_cast<size_t>(gridDim.x) * blockDim.x) {
      const size_t row = v / vpr;
      const int col = static_cast<int>(v % vpr) << 3;
      *reinterpret_cast<uint4*>(dst + row * cols + col) = *reinterpret_cast<const uint4*>(src + row * ld + col);
    }
  }
  cta_signal_all_and_wait(t, world, rank, slot0, target, wait_ns, status);
}

// ---------------------------------------------------------------------------
// Embedding: ids [B, S]; this rank owns vocabulary rows [v0, v1). For every token whose id
// it owns it writes the embedding row into the output shard of the rank that owns the
// token's sequence position: out_p[(s - p*S_shard), b, :]. Each output row is written by
// exactly one rank, so the "reduce" of the reference's reduce-scatter needs no additions.
__global__ void embedding_scatter_kernel(PeerTable t, const long long* __restrict__ ids,
                                         const __nv_bfloat16* __restrict__ W, int B, int S, int H, int v0, int v1,
                                         int world, int rank, int slot0, uint32_t target,
                                         unsigned long long wait_ns, uint32_t* status) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int S_shard = S / world;
  const int nvec = H >> 3;
  const long long total = static_cast<long long>(S) * B;
  for (long long tok = blockIdx.x * static_cast<long long>(warps_per_cta) + (threadIdx.x >> 5); tok < total;
       tok += static_cast<long long>(gridDim.x) * warps_per_cta) {
    const int s = static_cast<int>(tok / B);
    const int b = static_cast<int>(tok % B);
    const long long id = ids[static_cast<size_t>(b) * S + s];
    if (id < v0 || id >= v1) continue;
    const int owner = s / S_shard;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(t.buf[owner]) +
                         (static_cast<size_t>(s - owner * S_shard) * B + b) * H;
    const __nv_bfloat16* src = W + static_cast<size_t>(id - v0) * H;
    for (int v = lane; v < nvec; v += 32)
      *reinterpret_cast<uint4*>(dst + 8 * v) = *reinterpret_cast<const uint4*>(src + 8 * v);
  }
  cta_signal_all_and_wait(t, world, rank, slot0, target, wait_ns, status);
}

// ---------------------------------------------------------------------------
// Cross entropy: stats [M, 3] of this rank -> slot `rank` of every rank's [world, M, 3]
// buffer; after all ranks have delivered, combine into lse / loss (identical on all ranks).
__global__ void ce_exchange_kernel(PeerTable t, const float* __restrict__ stats, float* __restrict__ lse,
                                   float* __restrict__ loss, int M, int world, int rank, int slot0,
                                   uint32_t target, unsigned long long wait_ns, uint32_t* status) {
  const size_t n = static_cast<size_t>(M) * 3;
  for (int i = 0; i < world; ++i) {
    const int peer = (rank + i) % world;
    float* dst = static_cast<float*>(t.buf[peer]) + static_cast<size_t>(rank) * n;
    for (size_t k = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; k < n;
         k += static_cast<size_t>(gridDim.x) * blockDim.x)
      dst[k] = stats[k];
  }
  cta_signal_all_and_wait(t, world, rank, slot0, target, wait_ns, status);
  const float* all = static_cast<const float*>(t.buf[rank]);
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < M; row += gridDim.x * blockDim.x) {
    float gm = -INFINITY;
    for (int r = 0; r < world; ++r) gm = fmaxf(gm, all[(static_cast<size_t>(r) * M + row) * 3]);
    float gs = 0.f, tz = 0.f;
    for (int r = 0; r < world; ++r) {
      const float* st = all + (static_cast<size_t>(r) * M + row) * 3;
      gs += st[1] * __expf(st[0] - gm);
      tz += st[2];
    }
    const float l = gm + __logf(gs);
    lse[row] = l;
    loss[row] = l - tz;
  }
}

// ---------------------------------------------------------------------------
// Data-parallel optimizer. The flat gradient / parameter buffers are cut into buckets (runs of
// whole parameters, in the order the backward pass completes them); every rank owns one slice of
// EVERY bucket, and a rank's optimizer shard is the concatenation of its slices:
//
//   flat buffer : | bucket 0: r0 r1 .. | bucket 1: r0 r1 .. | ...      slice[b] elements per rank
//   shard of r  : | its slice of bucket 0 | its slice of bucket 1 | ...  (off[b] = start of slice b)
//
// so the gradient reduction of a bucket can start as soon as the backward pass has produced it,
// with equal work for every rank. Three kernels:
//   dp_push_grads   (per bucket, during backward, never waits): every rank copies the peers'
//                   slices of its local gradients into the owners' staging buffers over NVLink
//                   (copy engines) and signals
//   dp_sum_norm     (once, at the step): the owner waits for all pushes, sums the staged
//                   contributions in rank order (fp32, rounded to bf16 like a bf16 reduce-scatter)
//                   and publishes the squared norm of its shard to every rank
//   dp_adam_gather  (once): global-norm clip + AdamW on the fp32 shard + bf16 parameters stored
//                   into every rank's parameter buffer (all-gather by peer stores)
constexpr int MAX_BUCKETS = 16;
struct BucketTable {
  int nb;
  long long flat0[MAX_BUCKETS];    // first element of bucket b in the flat buffers
  long long slice[MAX_BUCKETS];    // elements per rank in bucket b (multiple of 8)
  long long off[MAX_BUCKETS + 1];  // first element of bucket b's slice in a shard; off[nb] = shard size
};

// staging buffer of rank r: [world (source)][shard] bf16. The pushes themselves are copy-engine
// transfers (cudaMemcpyAsync over NVLink, issued by gfs_dp_push_grads): they overlap the backward
// pass without taking SMs from its persistent kernels, which are sized to the whole GPU. This
// kernel, ordered after a bucket's copies on the same stream, tells every owner they have landed.
__global__ void dp_push_signal_kernel(PeerTable stage, int world, int rank, int slot) {
  if (threadIdx.x < world) red_release_sys_add_u32(stage.flags[threadIdx.x] + slot + rank, 1u);
}

template <int WORLD>
__global__ void __launch_bounds__(256)
dp_sum_norm_kernel(PeerTable stage, PeerTable norm, const __nv_bfloat16* __restrict__ grads, BucketTable bt,
                   __nv_bfloat16* __restrict__ reduced, int world_rt, int rank, int slot_push, uint32_t target_push,
                   int slot_norm, float* __restrict__ partials, unsigned int* __restrict__ ticket,
                   unsigned long long wait_ns, uint32_t* status) {
  const int world = WORLD > 0 ? WORLD : world_rt;
  constexpr int WMAX = WORLD > 0 ? WORLD : MAX_PEERS;
  // every peer's pushes of all buckets must have landed in our staging buffer (this rank's own
  // contribution is read straight from its gradient buffer: nothing is staged for it)
  if (threadIdx.x < world && threadIdx.x != rank)
    wait_flag_reached(stage.flags[rank] + slot_push + threadIdx.x, target_push, wait_ns, status,
                      0xD1000000u | (threadIdx.x << 4) | rank);
  __syncthreads();
  const __nv_bfloat16* mine = static_cast<const __nv_bfloat16*>(stage.buf[rank]);
  const long long shard = bt.off[bt.nb];
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = (WORLD > 0 && WORLD <= 4) ? 4 : 2;     // U x world 16-byte loads in flight per thread
  for (int b = 0; b < bt.nb; ++b) {
    const long long e_lo = bt.off[b];
    const long long nvec = (bt.off[b + 1] - e_lo) >> 3;
    const __nv_bfloat16* own = grads + bt.flat0[b] + rank * bt.slice[b];      // our slice of bucket b
    for (long long v0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v0 < nvec; v0 += U * stride) {
      uint4 in[U][WMAX];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * stride;
        if (v < nvec) {
#pragma unroll
          for (int r = 0; r < WMAX; ++r)
            if (r < world)
              in[u][r] = (r == rank) ? *reinterpret_cast<const uint4*>(own + (v << 3))
                                     : *reinterpret_cast<const uint4*>(mine + r * shard + e_lo + (v << 3));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long v = v0 + u * stride;
        if (v >= nvec) continue;
        float sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < WMAX; ++r) {
          if (r < world) {
            const float2 a = unpack_bf16x2(in[u][r].x), b2 = unpack_bf16x2(in[u][r].y),
                         c = unpack_bf16x2(in[u][r].z), d = unpack_bf16x2(in[u][r].w);
            sum[0] += a.x; sum[1] += a.y; sum[2] += b2.x; sum[3] += b2.y;
            sum[4] += c.x; sum[5] += c.y; sum[6] += d.x; sum[7] += d.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(sum[0], sum[1]);
        o.y = pack_bf16x2(sum[2], sum[3]);
        o.z = pack_bf16x2(sum[4], sum[5]);
        o.w = pack_bf16x2(sum[6], sum[7]);
        *reinterpret_cast<uint4*>(reduced + e_lo + (v << 3)) = o;
        const float2 a = unpack_bf16x2(o.x), b2 = unpack_bf16x2(o.y), c = unpack_bf16x2(o.z), d = unpack_bf16x2(o.w);
        acc += a.x * a.x + a.y * a.y + b2.x * b2.x + b2.y * b2.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
      }
    }
  }
  __shared__ float sm[8];
  __shared__ bool is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  acc = warp_sum(acc);
  if (lane == 0) sm[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = 0.f;
    for (int i = 0; i < 8; ++i) b += sm[i];
    partials[blockIdx.x] = b;
    __threadfence();
    is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0) {
    __threadfence();
    float total = 0.f;
    for (unsigned int i = 0; i < gridDim.x; ++i) total += reinterpret_cast<volatile float*>(partials)[i];
    *ticket = 0u;
    for (int r = 0; r < world; ++r) {
      static_cast<float*>(norm.buf[r])[rank] = total;
      red_release_sys_add_u32(norm.flags[r] + slot_norm + rank, 1u);
    }
  }
}

// Phase 2: wait for every rank's squared-norm, clip, AdamW on the fp32 master shard, and
// write the bf16 parameters into every rank's parameter buffer (all-gather by 16-byte peer
// stores, or one multicast store per vector when the buffers have a multicast address; the
// bucket table maps a shard position to its place in the flat buffer). Ends with a
// signal/wait so that when the kernel completes, this rank's own parameter buffer has
// received all shards.
__global__ void __launch_bounds__(256)
dp_adam_gather_kernel(PeerTable params, PeerTable norm, const __nv_bfloat16* __restrict__ reduced,
                      float* __restrict__ master, float* __restrict__ exp_avg, float* __restrict__ exp_avg_sq,
                      BucketTable bt, __nv_bfloat16* __restrict__ mc_params, int world, int rank, int slot_norm,
                      uint32_t target_norm,
                      int slot_param, uint32_t target_param, const float* __restrict__ extern_sumsq,
                      float* __restrict__ norm_out, AdamArgs a, unsigned long long wait_ns, uint32_t* status) {
  __shared__ float s_coef;
  if (threadIdx.x == 0) {
    float total = 0.f;
    if (extern_sumsq != nullptr) {
      total = *extern_sumsq;
    } else {
      for (int r = 0; r < world; ++r) {
        wait_flag_reached(norm.flags[rank] + slot_norm + r, target_norm, wait_ns, status,
                          0xD2000000u | (r << 4) | rank);
        total += reinterpret_cast<volatile float*>(norm.buf[rank])[r];
      }
    }
    const float nrm = sqrtf(total) * a.grad_scale;
    float coef = a.grad_scale;
    if (a.clip > 0.f && nrm > a.clip) coef *= a.clip / (nrm + 1e-6f);
    s_coef = coef;
    if (norm_out != nullptr && blockIdx.x == 0) *norm_out = nrm;
  }
  __syncthreads();
  const float coef = s_coef;
  float bc1, bc2_sqrt;
  adam_bias_corrections(a, bc1, bc2_sqrt);
  const float decay = 1.f - a.lr * a.weight_decay;
  const float step = a.lr / bc1;
  const float ob1 = 1.f - a.beta1, ob2 = 1.f - a.beta2;
  const long long nvec = bt.off[bt.nb] >> 3;          // 8 elements per thread and iteration
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i << 3;
    const uint4 gr = *reinterpret_cast<const uint4*>(reduced + e0);
    float g[8];
    {
      const float2 q0 = unpack_bf16x2(gr.x), q1 = unpack_bf16x2(gr.y), q2 = unpack_bf16x2(gr.z),
                   q3 = unpack_bf16x2(gr.w);
      g[0] = q0.x; g[1] = q0.y; g[2] = q1.x; g[3] = q1.y; g[4] = q2.x; g[5] = q2.y; g[6] = q3.x; g[7] = q3.y;
    }
    float4 p[2], m[2], v[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      p[h] = reinterpret_cast<const float4*>(master + e0)[h];
      m[h] = reinterpret_cast<const float4*>(exp_avg + e0)[h];
      v[h] = reinterpret_cast<const float4*>(exp_avg_sq + e0)[h];
    }
    float* pp = &p[0].x; float* mm = &m[0].x; float* vv = &v[0].x;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ge = g[e] * coef;
      pp[e] *= decay;
      mm[e] = a.beta1 * mm[e] + ob1 * ge;
      vv[e] = a.beta2 * vv[e] + ob2 * ge * ge;
      pp[e] -= step * (mm[e] / (sqrtf(vv[e]) / bc2_sqrt + a.eps));
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(master + e0)[h] = p[h];
      reinterpret_cast<float4*>(exp_avg + e0)[h] = m[h];
      reinterpret_cast<float4*>(exp_avg_sq + e0)[h] = v[h];
    }
    uint4 o;
    o.x = pack_bf16x2(pp[0], pp[1]);
    o.y = pack_bf16x2(pp[2], pp[3]);
    o.z = pack_bf16x2(pp[4], pp[5]);
    o.w = pack_bf16x2(pp[6], pp[7]);
    int b = 0;
    while (b + 1 < bt.nb && e0 >= bt.off[b + 1]) ++b;
    const long long flat = bt.flat0[b] + rank * bt.slice[b] + (e0 - bt.off[b]);
    if (mc_params != nullptr) {
      multimem_st_v4(mc_params + flat, o);          // NVSwitch delivers it to every rank's buffer
    } else {
      for (int q = 0; q < world; ++q) {
        const int r = (rank + 1 + q) % world;       // peers first: the remote stores leave early
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.buf[r]) + flat) = o;
      }
    }
  }
  cta_signal_all_and_wait(params, world, rank, slot_param, target_param, wait_ns, status);
}

int fill_table(PeerTable& t, const unsigned long long* bufs, const unsigned long long* flags, int world) {
  if (world < 1 || world > MAX_PEERS) return -1;
  for (int i = 0; i < MAX_PEERS; ++i) {
    t.buf[i] = i < world && bufs ? reinterpret_cast<void*>(bufs[i]) : nullptr;
    t.flags[i] = i < world && flags ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
  }
  return 0;
}

unsigned long long limit_of(long long wait_ns) {
  return wait_ns > 0 ? static_cast<unsigned long long>(wait_ns) : 20000000000ull;
}

int resident_grid(int want) { return std::max(1, std::min(want, gfs_host::sm_count() * 2)); }

}  // namespace

extern "C" {

// In every function: peer_bufs / peer_flags are host arrays of `world` device pointers (this
// rank's entry included); buffer tables carry one more entry, [world]: the multicast address of
// the same symmetric buffers (0 when there is none), used where a kernel says so; slot0 is the first of `world` consecutive uint32 counters reserved
// for the call site inside each rank's flag array; *target_inout is the cumulative count and
// is advanced by the call (identically on all ranks). Grids are sized so that all CTAs are
// co-resident, because CTAs wait for signals produced by other GPUs' CTAs.

int gfs_symm_barrier(const unsigned long long* peer_flags, int world, int rank, int slot0,
                     unsigned int* target_inout, long long wait_ns, void* stream) {
  PeerTable t;
  if (fill_table(t, nullptr, peer_flags, world)) return -1;
  *target_inout += 1;
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, world, rank, slot0, *target_inout,
                                                                      limit_of(wait_ns), gfs_host::status_words());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_allgather(const void* src, int rows, int cols, int ld, const unsigned long long* peer_bufs,
                  const unsigned long long* peer_flags, int world, int rank, int slot0, unsigned int* target_inout,
                  long long wait_ns, void* stream) {
  PeerTable t;
  if (fill_table(t, peer_bufs, peer_flags, world) || (cols & 7) || (ld & 7)) return -1;
  const size_t total = static_cast<size_t>(rows) * (cols >> 3);
  const int grid = resident_grid(static_cast<int>((total + 255) / 256));
  *target_inout += static_cast<unsigned int>(grid);
  allgather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      t, static_cast<const __nv_bfloat16*>(src), rows, cols, ld, world, rank, slot0, *target_inout, limit_of(wait_ns),
      gfs_host::status_words());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_embedding_scatter(const void* ids, const void* W, int B, int S, int H, int v0, int v1,
                          const unsigned long long* peer_out, const unsigned long long* peer_flags, int world,
                          int rank, int slot0, unsigned int* target_inout, long long wait_ns, void* stream) {
  PeerTable t;
  if (fill_table(t, peer_out, peer_flags, world) || (H & 7) || (S % world)) return -1;
  const long long tokens = static_cast<long long>(S) * B;
  const int grid = resident_grid(static_cast<int>((tokens + 7) / 8));
  *target_inout += static_cast<unsigned int>(grid);
  embedding_scatter_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      t, static_cast<const long long*>(ids), static_cast<const __nv_bfloat16*>(W), B, S, H, v0, v1, world, rank, slot0,
      *target_inout, limit_of(wait_ns), gfs_host::status_words());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

int gfs_ce_exchange(const void* stats, void* lse, void* loss, int M, const unsigned long long* peer_bufs,
                    const unsigned long long* peer_flags, int world, int rank, int slot0,
                    unsigned int* target_inout, long long wait_ns, void* stream) {
  PeerTable t;
  if (fill_table(t, peer_bufs, peer_flags, world)) return -1;
  const int grid = resident_grid((M * 3 + 255) / 256);
  *target_inout += static_cast<unsigned int>(grid);
  ce_exchange_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      t, static_cast<const float*>(stats), static_cast<float*>(lse), static_cast<float*>(loss), M, world, rank, slot0,
      *target_inout, limit_of(wait_ns), gfs_host::status_words());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// ---- data-parallel optimizer (see the kernels above) ----
// A bucket table is passed as three host arrays of nb (off: nb + 1) entries, in elements.
static int fill_buckets(BucketTable& bt, int nb, const long long* flat0, const long long* slice, const long long* off) {
  if (nb < 1 || nb > MAX_BUCKETS) return -1;
  bt.nb = nb;
  for (int b = 0; b < nb; ++b) {
    if ((flat0[b] & 7) || (slice[b] & 7) || (off[b] & 7) || slice[b] <= 0) return -1;
    bt.flat0[b] = flat0[b];
    bt.slice[b] = slice[b];
    bt.off[b] = off[b];
  }
  if (off[nb] & 7) return -1;
  bt.off[nb] = off[nb];
  return 0;
}

// Pushes bucket `b` of the local gradient buffer: slice r goes to rank r's staging buffer
// (peer_stage[r] = rank r's [world][shard] bf16 buffer), at [this rank][off[b] ...), by one
// copy-engine transfer per destination (peers first), followed by a one-warp kernel that signals
// the owners. Never waits; meant for a side stream while the backward pass continues.
// *target_inout: cumulative number of signals each owner must see from each source (+1 per call).
int gfs_dp_push_grads(const void* grads, const unsigned long long* peer_stage, const unsigned long long* peer_flags,
                      int nb, const long long* flat0, const long long* slice, const long long* off, int b, int world,
                      int rank, int slot_push, unsigned int* target_inout, void* stream_) {
  PeerTable st;
  BucketTable bt;
  if (fill_table(st, peer_stage, peer_flags, world) || fill_buckets(bt, nb, flat0, slice, off)) return -1;
  if (b < 0 || b >= nb) return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const __nv_bfloat16* g = static_cast<const __nv_bfloat16*>(grads);
  const size_t bytes = static_cast<size_t>(bt.slice[b]) * sizeof(__nv_bfloat16);
  for (int q = 0; q + 1 < world; ++q) {          // peers only: the owner reads its own slice in place
    const int dst = (rank + 1 + q) % world;
    __nv_bfloat16* to = static_cast<__nv_bfloat16*>(st.buf[dst]) + rank * bt.off[nb] + bt.off[b];
    if (cudaMemcpyAsync(to, g + bt.flat0[b] + dst * bt.slice[b], bytes, cudaMemcpyDeviceToDevice, stream) !=
        cudaSuccess)
      return -12;
  }
  *target_inout += 1u;
  dp_push_signal_kernel<<<1, 32, 0, stream>>>(st, world, rank, slot_push);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// scratch: fp32 [2 * SMs + 8] zero-initialised once (per-CTA partials followed by the ticket);
// gfs_dp_reduce_norm_scratch_floats() gives its size.
int gfs_dp_reduce_norm_scratch_floats() { return gfs_host::sm_count() * 2 + 8; }

// Sums the gradient contributions of all ranks (the peers' from the staging buffer, this rank's
// own from `grads`) into `reduced` (this rank's shard) once every push has arrived (target_push = the value gfs_dp_push_grads left in its counter), and
// publishes the shard's squared norm to every rank (peer_norm_slots[r][rank], flag slot_norm).
int gfs_dp_sum_norm(const void* grads, const unsigned long long* peer_stage, const unsigned long long* peer_flags,
                    const unsigned long long* peer_norm_slots, void* reduced, int nb, const long long* flat0,
                    const long long* slice, const long long* off, int world, int rank, int slot_push,
                    unsigned int target_push, int slot_norm, unsigned int* target_norm_inout, void* scratch,
                    long long wait_ns, void* stream) {
  PeerTable st, nm;
  BucketTable bt;
  if (fill_table(st, peer_stage, peer_flags, world) || fill_table(nm, peer_norm_slots, peer_flags, world)) return -1;
  if (fill_buckets(bt, nb, flat0, slice, off)) return -1;
  const long long shard_numel = bt.off[nb];
  const int grid = resident_grid(static_cast<int>(((shard_numel >> 3) + 2 * 256 - 1) / (2 * 256)));
  *target_norm_inout += 1;
  float* partials = static_cast<float*>(scratch);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(partials + gfs_host::sm_count() * 2 + 4);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* red = static_cast<__nv_bfloat16*>(reduced);
#define GFS_SUM_NORM(W)                                                                                          \
  dp_sum_norm_kernel<W><<<grid, 256, 0, s>>>(st, nm, static_cast<const __nv_bfloat16*>(grads), bt, red, world,   \
                                             rank, slot_push, target_push, slot_norm, partials, ticket,          \
                                             limit_of(wait_ns), gfs_host::status_words())
  if (world == 2) GFS_SUM_NORM(2);
  else if (world == 4) GFS_SUM_NORM(4);
  else if (world == 8) GFS_SUM_NORM(8);
  else GFS_SUM_NORM(0);
#undef GFS_SUM_NORM
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// extern_sumsq: device scalar with the global squared gradient norm computed elsewhere
// (e.g. reduced over tensor-parallel ranks as well), or null to use the per-rank values
// exchanged by gfs_dp_sum_norm (target_norm = the value that call left in its counter).
// step_dev: as in gfs_adamw_step (loss_optim.cu).
int gfs_dp_adam_gather(const unsigned long long* peer_params, const unsigned long long* peer_flags,
                       const unsigned long long* peer_norm_slots, const void* reduced, void* master, void* exp_avg,
                       void* exp_avg_sq, int nb, const long long* flat0, const long long* slice, const long long* off,
                       int world, int rank, int slot_norm, unsigned int target_norm, int slot_param,
                       unsigned int* target_param_inout, const void* extern_sumsq, void* norm_out, float lr,
                       double beta1, double beta2, float eps, float weight_decay, float bias_corr1,
                       float bias_corr2_sqrt, float clip, float grad_scale, const void* step_dev, long long wait_ns,
                       void* stream) {
  PeerTable pr, nm;
  BucketTable bt;
  if (fill_table(pr, peer_params, peer_flags, world) || fill_table(nm, peer_norm_slots, peer_flags, world)) return -1;
  if (fill_buckets(bt, nb, flat0, slice, off)) return -1;
  const long long shard_numel = bt.off[nb];
  const int grid = resident_grid(static_cast<int>(((shard_numel >> 3) + 255) / 256));
  *target_param_inout += static_cast<unsigned int>(grid);
  AdamArgs a{lr, static_cast<float>(beta1), static_cast<float>(beta2), eps, weight_decay, bias_corr1,
             bias_corr2_sqrt, clip, grad_scale, static_cast<const float*>(step_dev), beta1, beta2};
  dp_adam_gather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pr, nm, static_cast<const __nv_bfloat16*>(reduced), static_cast<float*>(master), static_cast<float*>(exp_avg),
      static_cast<float*>(exp_avg_sq), bt, reinterpret_cast<__nv_bfloat16*>(peer_params[world]), world, rank,
      slot_norm, target_norm, slot_param, *target_param_inout,
      static_cast<const float*>(extern_sumsq), static_cast<float*>(norm_out), a, limit_of(wait_ns),
      gfs_host::status_words());
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // extern "C"
