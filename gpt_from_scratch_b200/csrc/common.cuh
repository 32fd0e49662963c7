// Shared device/host helpers for the sm_100a kernels of this library.
//
// Contents:
//   * status word protocol (every bounded wait that gives up records a code here
//     and the kernel still runs to completion, so the CUDA context stays usable)
//   * mbarrier, TMA (cp.async.bulk.tensor, plain non-cluster-broadcast loads only),
//     tcgen05 (alloc / mma / commit / ld / fences) inline-PTX wrappers
//   * UMMA shared-memory and instruction descriptor builders for bf16 operands
//     in the 128-byte-swizzled canonical layouts (K-major and MN-major)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gfs {

// ----------------------------------------------------------------------------
// Status codes written (first writer wins) to status[0]; status[1] gets a detail.
// ----------------------------------------------------------------------------
enum StatusCode : uint32_t {
  STATUS_OK = 0,
  STATUS_TIMEOUT_PIPE_FULL = 1,    // consumer waited for a TMA stage
  STATUS_TIMEOUT_PIPE_EMPTY = 2,   // producer waited for a free stage
  STATUS_TIMEOUT_TMEM_FULL = 3,    // epilogue waited for the accumulator
  STATUS_TIMEOUT_TMEM_EMPTY = 4,   // MMA warp waited for a drained accumulator
  STATUS_TIMEOUT_SOFTMAX = 5,      // attention role hand-off
  STATUS_TIMEOUT_PEER_FLAG = 6,    // cross-GPU flag never arrived
  STATUS_TIMEOUT_GRID_BARRIER = 7, // intra-kernel grid barrier
  STATUS_BAD_ARGUMENT = 8,
  STATUS_TIMEOUT_TEST_FLAG = 9,    // the wait-probe kernel (a flag nothing sets)
};

#ifndef GFS_WAIT_LIMIT_NS
#define GFS_WAIT_LIMIT_NS 2000000000ull  // 2 s for waits inside one kernel
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Per-CTA abort context: once any wait in the CTA gives up, every later wait
// returns immediately so the CTA drains and exits.
struct WaitCtx {
  volatile uint32_t* abort_flag;  // shared memory word, zero-initialised
  uint32_t* status;               // global status words (may be nullptr)
  uint64_t limit_ns;
};

__device__ __forceinline__ void record_status(uint32_t* status, uint32_t code, uint32_t detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0u, code) == 0u) status[1] = detail;
  }
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking poll (try_wait may suspend the thread for a hardware-defined time before it
// answers; a loop that watches several barriers needs the immediate form).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false if the wait was abandoned (status recorded). The global timer
// is slow to read, so it is only consulted every 4096 failed polls; the first reading
// starts the clock.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*ctx.abort_flag) return false;
  uint32_t it = 0;
  uint64_t t0 = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (((++it) & 0xfffu) == 0u) {
      if (*ctx.abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > ctx.limit_ns) {
        *ctx.abort_flag = 1u;
        record_status(ctx.status, code, (blockIdx.x << 8) | (threadIdx.x >> 5));
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// TMA (bulk tensor copies global -> shared of this CTA, completion on an mbarrier)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 1-D bulk copy global -> shared of this CTA (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Generic-proxy writes to shared memory that the async proxy (UMMA / TMA) will read.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Generic-proxy global writes (possibly by a peer GPU) that a later TMA load will read.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// ----------------------------------------------------------------------------
// tcgen05 / TMEM
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {  // whole warp
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Warp-collective variants: ALL 32 lanes of the issuing warp call them (converged) and one
// elected lane issues. Running the issuing loop on the whole warp keeps its address and
// descriptor arithmetic warp-uniform, which the compiler maps to the uniform datapath; inside
// an `if (lane == 0)` branch every tcgen05.mma operand has to be moved over from the vector
// registers first, which makes the issue itself the bottleneck for short (N = 64) MMAs
// (measured: 8 MMAs with stage-dependent descriptors issue in 261 cycles this way, 497 from a
// single-lane branch). elect.sync picks the same lane for the same mask every time, so the
// commits below track the MMAs issued by the same thread.
__device__ __forceinline__ void umma_ss_e(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_e(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit_e(uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar))
      : "memory");
}
// Arrive on an mbarrier when all previously issued MMAs of this thread are done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (base+t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M = 128 rows on the 128 lanes, K elements
// packed two bf16 per 32-bit column) is read from tensor memory.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns from registers into tensor memory.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Same wait, but naming the destination registers so the compiler cannot schedule their
// consumers above it when loads and arithmetic are software-pipelined.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                 "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                 "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_for16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                 "+r"(r[15])
               :
               : "memory");
}

// ----------------------------------------------------------------------------
// UMMA descriptors (bf16, 128-byte swizzle)
// ----------------------------------------------------------------------------
// Shared-memory matrix descriptor, 64 bits:
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1 (Blackwell)
//   [61,64) layout type: 2 = 128-byte swizzle
// K-major tile (rows of 64 bf16 = 128 B, 8-row groups 1024 B apart): SBO = 1024, LBO unused.
// MN-major tile (rows = K index, each row 64 MN-elements = 128 B; 8-row groups
// 1024 B apart; the next 64 MN-elements start `lbo_bytes` further): SBO = 1024, LBO = lbo_bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   [4,6) D format (1 = f32)  [7,10) A format (1 = bf16)  [10,13) B format (1 = bf16)
//   [15] A major (1 = MN)     [16] B major (1 = MN)       [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Byte offset of element (row, col) inside one 128B-swizzled block whose rows are
// 64 bf16 (128 B) wide and whose base is 1024-byte aligned: the 16-byte chunk
// index is XORed with (row mod 8).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t col) {
  return row * 128u + ((((col >> 3) ^ (row & 7u)) & 7u) << 4) + ((col & 7u) << 1);
}

// ----------------------------------------------------------------------------
// misc
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float fast_exp2(float x) {  // ex2.approx: exp2(-inf) = +0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Programmatic dependent launch (see gfs_host::launch_pdl). pdl_wait(): returns once the preceding
// kernel of the stream has completed and its writes are visible (a no-op for a normal launch);
// nothing before it may touch global memory that another kernel writes or reads. pdl_trigger():
// this CTA no longer objects to the next kernel's CTAs being scheduled on SMs that become free.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ----------------------------------------------------------------------------
// Cross-GPU flags (peer memory over NVLink). Counters only grow; a waiter compares
// against a cumulative target, so no flag is ever reset.
//
// Layout of a rank's flag array: FLAG_SLOTS counters followed by FLAG_SLOTS "base" words, one per
// counter. The value a counter must reach is  base[slot] + target  where `target` is the kernel
// argument the host computed. In ordinary (eager) launches the base words are zero and `target` is
// the host's cumulative count. A step captured in a CUDA graph replays with frozen kernel
// arguments: there `target` is the count relative to the start of the step and the last node of
// the graph adds the step's total to the base words, so every replay waits for the right value.
// Base words are local (only this rank's kernels read or write them).
// ----------------------------------------------------------------------------
constexpr uint32_t FLAG_SLOTS = 8192;
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// One 16-byte store to a multicast address: NVSwitch writes it to the same offset of every rank's
// copy of the symmetric buffer (this rank's own included), so an all-gather leaves the GPU once
// instead of once per peer. Ordered like any other store by the fences / release that follow it.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void red_release_gpu_add_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *p has reached `target` (wrap-safe). On expiry records
// STATUS_TIMEOUT_PEER_FLAG with `detail` and returns false.
__device__ __forceinline__ bool wait_flag_reached(const uint32_t* p, uint32_t target, uint64_t limit_ns,
                                                  uint32_t* status, uint32_t detail) {
  uint32_t it = 0;
  uint64_t t0 = 0;
  target += *reinterpret_cast<const volatile uint32_t*>(p + FLAG_SLOTS);   // this counter's base word
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) >= 0) return true;
    __nanosleep(64);
    if (((++it) & 0x3ffu) == 0u) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        record_status(status, STATUS_TIMEOUT_PEER_FLAG, detail);
        return false;
      }
    }
  }
}
// Hyper-parameters of one AdamW update. The bias corrections are either given by the host
// (bias_corr1 = 1 - beta1^t, bias_corr2_sqrt = sqrt(1 - beta2^t)) or, when `step_dev` is set,
// computed by the kernel from the step count t kept in device memory, so that a launch captured
// in a CUDA graph (frozen arguments) still sees the current step on every replay.
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_corr1, bias_corr2_sqrt;
  float clip, grad_scale;
  const float* step_dev;
  double beta1_d, beta2_d;
};
// Called by all threads of the CTA (contains a __syncthreads when step_dev is set).
__device__ __forceinline__ void adam_bias_corrections(const AdamArgs& a, float& bc1, float& bc2_sqrt) {
  bc1 = a.bias_corr1;
  bc2_sqrt = a.bias_corr2_sqrt;
  if (a.step_dev != nullptr) {
    __shared__ float s_bc[2];
    if (threadIdx.x == 0) {
      const double t = static_cast<double>(*a.step_dev);
      s_bc[0] = static_cast<float>(1.0 - pow(a.beta1_d, t));
      s_bc[1] = static_cast<float>(sqrt(1.0 - pow(a.beta2_d, t)));
    }
    __syncthreads();
    bc1 = s_bc[0];
    bc2_sqrt = s_bc[1];
  }
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads);

// First step of a fused all-gather -> GEMM: the calling threads (`nthreads` of this CTA, the caller
// being number `tid`; all of them must call) copy this CTA's slice of the local shard into every
// rank's gathered buffer (own rank first, then the peers in ring order) with 16-byte stores and,
// per destination, bump that rank's counter for this source once the slice is written.
// `bar_id` is a named barrier reserved for these threads.
template <typename Comm>
__device__ __forceinline__ void ag_push_rows(const Comm& c, int tid, int nthreads, int bar_id) {
  const int rpc = (c.rows_per_rank + gridDim.x - 1) / gridDim.x;
  const int r0 = min(c.rows_per_rank, static_cast<int>(blockIdx.x) * rpc);
  const int r1 = min(c.rows_per_rank, r0 + rpc);
  const int vpr = c.ag_cols >> 3;
  const int nvec = (r1 - r0) * vpr;
  if (c.mc_buf != nullptr) {
    // multicast: one store per vector reaches every rank's gathered buffer through the switch
    __nv_bfloat16* dst = c.mc_buf + static_cast<size_t>(c.rank) * c.rows_per_rank * c.ag_cols;
    for (int v = tid; v < nvec; v += nthreads * 4) {
      uint4 tmp[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vv = v + u * nthreads;
        if (vv < nvec) {
          const int row = r0 + vv / vpr;
          tmp[u] = *reinterpret_cast<const uint4*>(c.ag_src + static_cast<size_t>(row) * c.ag_ld + (vv % vpr) * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vv = v + u * nthreads;
        if (vv < nvec) {
          const int row = r0 + vv / vpr;
          multimem_st_v4(dst + static_cast<size_t>(row) * c.ag_cols + (vv % vpr) * 8, tmp[u]);
        }
      }
    }
    // (no fence per thread: the barrier orders every thread's stores before the signalling threads'
    // release, which is cumulative; a system-scope fence costs microseconds)
    named_barrier_sync(bar_id, nthreads);
    if (tid < c.world) red_release_sys_add_u32(c.peer_flags[tid] + c.rank, 1u);
    return;
  }
  // The system-scope release that publishes the rows costs microseconds, so there is one for all
  // destinations, not one per destination: store to every rank (peers first, the rows are re-read
  // from cache), CTA barrier, then one thread per destination bumps its counter with release
  // semantics (cumulative over the stores the barrier ordered before it).
  for (int i = 1; i <= c.world; ++i) {
    const int peer = (c.rank + i) % c.world;
    __nv_bfloat16* dst = c.peer_buf[peer] + static_cast<size_t>(c.rank) * c.rows_per_rank * c.ag_cols;
    for (int v = tid; v < nvec; v += nthreads * 4) {
      uint4 tmp[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vv = v + u * nthreads;
        if (vv < nvec) {
          const int row = r0 + vv / vpr;
          tmp[u] = *reinterpret_cast<const uint4*>(c.ag_src + static_cast<size_t>(row) * c.ag_ld + (vv % vpr) * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vv = v + u * nthreads;
        if (vv < nvec) {
          const int row = r0 + vv / vpr;
          *reinterpret_cast<uint4*>(dst + static_cast<size_t>(row) * c.ag_cols + (vv % vpr) * 8) = tmp[u];
        }
      }
    }
  }
  named_barrier_sync(bar_id, nthreads);
  if (tid < c.world) red_release_sys_add_u32(c.peer_flags[tid] + c.rank, 1u);
}

// Final step of a fused GEMM -> reduce-scatter: out[row, :] = sum over source ranks of the staged
// bf16 partial rows (in rank order: deterministic) + optional residual, rounded once. `stage` is
// this rank's staging area [world][rows][N]. The vectors (8 columns each) are dealt to
// `nthreads_total` threads of the whole grid, of which the caller is number `tid_global`. All of a
// step's loads (U vectors x WORLD sources + U residual vectors) are issued before the first sum, so
// a thread has U * (WORLD + 1) independent 16-byte loads in flight and the pass runs at memory
// speed; with the source loop left to run time the loads of one vector serialise (one memory
// latency per source), which made this pass the longest part of the small reduce-scatter GEMMs.
template <int WORLD, int U>
__device__ __forceinline__ void rs_reduce_rows_t(const __nv_bfloat16* __restrict__ stage, int rows, int N,
                                                 const __nv_bfloat16* __restrict__ res, int ld_res,
                                                 __nv_bfloat16* __restrict__ out, int ld_out, uint32_t tid_global,
                                                 uint32_t nthreads_total) {
  const uint32_t vpr = static_cast<uint32_t>(N) >> 3;
  const uint32_t total = static_cast<uint32_t>(rows) * vpr;       // < 2^32: rows * N / 8 of one row chunk
  const size_t chunk_elems = static_cast<size_t>(rows) * N;
  for (uint32_t v0 = tid_global; v0 < total; v0 += nthreads_total * U) {
    uint4 in[U][WORLD];
    uint4 rr[U];
    uint32_t row[U], col[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t v = v0 + static_cast<uint32_t>(u) * nthreads_total;
      const bool live = v < total;
      row[u] = live ? v / vpr : 0u;
      col[u] = live ? (v - row[u] * vpr) << 3 : 0u;
      const __nv_bfloat16* src0 = stage + static_cast<size_t>(row[u]) * N + col[u];
#pragma unroll
      for (int s = 0; s < WORLD; ++s) in[u][s] = *reinterpret_cast<const uint4*>(src0 + s * chunk_elems);
      rr[u] = (res != nullptr) ? *reinterpret_cast<const uint4*>(res + static_cast<size_t>(row[u]) * ld_res + col[u])
                               : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + static_cast<uint32_t>(u) * nthreads_total >= total) continue;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < WORLD; ++s) {
        const float2 a = unpack_bf16x2(in[u][s].x), b = unpack_bf16x2(in[u][s].y), c = unpack_bf16x2(in[u][s].z),
                     d = unpack_bf16x2(in[u][s].w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
      const float2 a = unpack_bf16x2(rr[u].x), b = unpack_bf16x2(rr[u].y), c = unpack_bf16x2(rr[u].z),
                   d = unpack_bf16x2(rr[u].w);
      uint4 o;
      o.x = pack_bf16x2(acc[0] + a.x, acc[1] + a.y);
      o.y = pack_bf16x2(acc[2] + b.x, acc[3] + b.y);
      o.z = pack_bf16x2(acc[4] + c.x, acc[5] + c.y);
      o.w = pack_bf16x2(acc[6] + d.x, acc[7] + d.y);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(row[u]) * ld_out + col[u]) = o;
    }
  }
}

__device__ __forceinline__ void rs_reduce_rows(const __nv_bfloat16* __restrict__ stage, int world, int rows, int N,
                                               const __nv_bfloat16* __restrict__ res, int ld_res,
                                               __nv_bfloat16* __restrict__ out, int ld_out, size_t tid_global,
                                               size_t nthreads_total) {
  const uint32_t t = static_cast<uint32_t>(tid_global), n = static_cast<uint32_t>(nthreads_total);
  switch (world) {
    case 2: rs_reduce_rows_t<2, 4>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
    case 3: rs_reduce_rows_t<3, 2>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
    case 4: rs_reduce_rows_t<4, 2>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
    case 5: rs_reduce_rows_t<5, 2>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
    case 6: rs_reduce_rows_t<6, 2>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
    case 7: rs_reduce_rows_t<7, 2>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
    default: rs_reduce_rows_t<8, 2>(stage, rows, N, res, ld_res, out, ld_out, t, n); break;
  }
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Counted arrival without waiting: the warps that call bar.sync on the same barrier are released
// once `nthreads` threads (arrivals + waiters) have reached it.
__device__ __forceinline__ void named_barrier_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace gfs

// ----------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------
namespace gfs_host {

// Encode a tiled bf16 tensor map with 128-byte swizzle. dims/strides are innermost
// first; strides[0] is implied (2 bytes). Returns 0 on success.
int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box);
// Cached 2-D variant: tensor [rows, cols] with row pitch ld (elements), box [box_rows, 64 cols].
const CUtensorMap* tmap_2d_cached(const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                                  uint32_t box_rows, uint32_t box_cols);
const CUtensorMap* tmap_nd_cached(const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                                  const uint32_t* box);
// Device status words owned by the library (allocated on first use per device).
uint32_t* status_words();
int sm_count();
// Programmatic dependent launch allowed (GFS_PDL, default on).
bool pdl_enabled();

// Launch with programmatic stream serialization: the kernel's CTAs may become resident and run
// their set-up while the preceding kernel of the stream drains; the kernel must call
// gfs::pdl_wait() before its first access to global memory. Inside a stream capture the
// dependency becomes a programmatic edge of the graph.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace gfs_host
