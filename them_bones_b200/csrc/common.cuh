// Shared device helpers for the sm_100a kernels: mbarrier (bounded waits), TMA bulk-tensor copies, tcgen05 MMA / TMEM
// access, UMMA shared-memory and instruction descriptors.
//
// Every wait on an mbarrier is bounded: when the cycle budget runs out the waiter raises a CTA-wide abort flag, records
// an error code in a host-visible word and returns false; callers leave their role loops, fall through to the common
// tear-down (TMEM is freed, the CTA exits) and the host raises after reading the word.  Nothing spins forever and
// nothing traps.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bones {

constexpr long long kWaitLimitCycles = 3000000000LL;   // ~1.5 s at 1.9 GHz

enum ErrCode : int {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 1,      // consumer never saw a TMA stage land
  ERR_WAIT_EMPTY = 2,     // producer never got a stage back
  ERR_WAIT_TMEM_FULL = 3, // epilogue never saw the accumulator commit
  ERR_WAIT_TMEM_EMPTY = 4,
  ERR_WAIT_PEER = 5,      // a flag written by another GPU never arrived
  ERR_BAD_ARG = 6,
  ERR_WAIT_AUX = 7,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// The wait carries a suspend-time hint: a warp whose barrier is not ready yet is parked by the hardware (and woken when
// the phase completes) instead of coming back to re-issue the instruction every few hundred cycles.  Waiting warps share
// their scheduler with the one thread that issues a CTA's MMAs, so every slot they do not take is one it can use.
constexpr uint32_t kWaitHintNs = 2000;
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return ok != 0;
}
// One lane of a fully active warp (`elect.sync`).  The role loops of the tensor-core kernels run on all 32 lanes with
// warp-uniform operands and issue their `tcgen05` / TMA instructions from the elected lane: those instructions take
// their operands from uniform registers, and operands computed under a `lane == 0` branch live in per-thread
// registers and are moved over one by one (measured: about 80 clocks per `tcgen05.mma` issued that way).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// Lane 0's value on every lane.  Besides handing a value round, the shuffle tells the compiler that what follows from it
// (loop bounds, stage indices, descriptors) is warp-uniform.
__device__ __forceinline__ int warp_uniform(int v) { return __shfl_sync(0xffffffffu, v, 0); }
// Bounded wait.  `abort_flag` lives in shared memory and is raised by whichever role gives up first.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      if (err) atomicCAS(err, 0, code);
      return false;
    }
  }
}

// Dynamic work distribution for persistent kernels: the CTA's producer thread draws item numbers from a global counter
// (zeroed by the host before the launch) and hands them to the CTA's other roles through a four-slot ring in shared
// memory (four mbarriers of count 1 at `bars`, four ints at `slots`).  A role may run at most three items behind the
// producer.  -1 ends the walk.
__device__ __forceinline__ int item_publish(uint32_t bars, volatile int* slots, int it, int* counter, int total) {
  const int w = atomicAdd(counter, 1);
  const int v = w < total ? w : -1;
  slots[it & 3] = v;
  mbar_arrive(bars + 8u * (uint32_t)(it & 3));
  return v;
}
__device__ __forceinline__ int item_take(uint32_t bars, volatile int* slots, int it, volatile int* abort_flag, int* err) {
  if (!mbar_wait(bars + 8u * (uint32_t)(it & 3), (uint32_t)((it >> 2) & 1), abort_flag, err, ERR_WAIT_AUX)) return -1;
  return slots[it & 3];
}

// ---------------------------------------------------------------------------------------------------------------
// TMA (bulk tensor copies; no cluster multicast anywhere)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Plain (untiled) bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {                         // one thread
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from TMEM (e.g. softmax probabilities written back as bf16), B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same two MMAs with the shared-memory descriptors passed as (low, high) 32-bit halves.  A single thread issues
// every MMA of a CTA, and its instruction stream is what limits 128 x 128 x 16 MMAs (64 tensor-pipe cycles each): with
// the high half a compile-time constant and the low half `base + constant` per UMMA_K step, an MMA costs an integer add
// per operand instead of a descriptor build.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo_bytes, uint32_t layout) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | ((layout & 7u) << 29);
}
__device__ __forceinline__ void umma_f16_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ts_lh(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Block-scaled MXFP8: E4M3/E5M2 elements, UE8M0 scale per 32 elements of K, scales resident in TMEM.
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// shared -> TMEM copy of 32 lanes x 128 bits replicated to the four 32-lane sub-partitions (scale factors)
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

#define BONES_TMEM_LD32(taddr, r)                                                                                        \
  asm volatile(                                                                                                          \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                          \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "  \
      "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                                                                  \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),       \
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),           \
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),          \
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])                        \
      : "r"(taddr)                                                                                                       \
      : "memory")

#define BONES_TMEM_ST32(taddr, r)                                                                                        \
  asm volatile(                                                                                                          \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "                                                                   \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "  \
      "%24, %25, %26, %27, %28, %29, %30, %31};" ::"r"(r[0]),                                                            \
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),      \
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),         \
      "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),         \
      "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)                                                                     \
      : "memory")

#define BONES_TMEM_LD16(taddr, r)                                                                                        \
  asm volatile(                                                                                                          \
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "                                                                          \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"                                   \
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),       \
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])                         \
      : "r"(taddr)                                                                                                       \
      : "memory")

#define BONES_TMEM_ST16(taddr, r)                                                                                        \
  asm volatile(                                                                                                          \
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "                                                                   \
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),                             \
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),      \
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)                                             \
      : "memory")

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  Fields (bits): start address >> 4 [0,14), leading byte offset >> 4
// [16,30), stride byte offset >> 4 [32,46), descriptor version 1 at [46,48), layout type [61,64) (2 = SWIZZLE_128B,
// 0 = no swizzle).
__host__ __device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7u) << 61;
  return d;
}
constexpr uint32_t kLayoutSw128 = 2;
constexpr uint32_t kLayoutNone = 0;

// Instruction descriptor for kind::f16 with fp32 accumulation.  fmt: 0 = fp16, 1 = bf16.  major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n, uint32_t fmt, uint32_t a_major, uint32_t b_major) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_major << 15) | (b_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Instruction descriptor for kind::mxf8f6f4.block_scale with UE8M0 scales.  a_fmt/b_fmt: 0 = E4M3, 1 = E5M2.
__host__ __device__ constexpr uint32_t umma_idesc_mxf8(uint32_t m, uint32_t n, uint32_t a_fmt, uint32_t b_fmt, uint32_t a_major,
                                                       uint32_t b_major, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_major << 15) | (b_major << 16) | ((n >> 3) << 17) | (1u << 23) |
         ((m >> 4) << 24) | (a_sf_id << 29);
}

// ---------------------------------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
// 256-bit global accesses (one full 32-byte sector per thread); the address must be 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x),
               "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}
__device__ __forceinline__ void ld_global_v8(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(p)
               : "memory");
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

// ---------------------------------------------------------------------------------------------------------------
// Debug-bounds build (-DBONES_DEBUG_BOUNDS, library libbones_b200_dbg.so): every data-dependent index (token ids, slot
// tables, hashed row ids, staging positions) is checked against the extent it addresses; a miss is counted, its value
// and source line are kept, and the access is skipped.  No memory checker runs on the machines this library is
// developed on; this build is its stand-in for the index-driven kernels.  The release build compiles the checks away.
// ---------------------------------------------------------------------------------------------------------------
#ifdef BONES_DEBUG_BOUNDS
static __device__ int g_bounds_hits = 0;
static __device__ long long g_bounds_last[2] = {0, 0};
__device__ __forceinline__ bool bones_index_ok(long long i, long long lo, long long hi, int line) {
  if (i >= lo && i < hi) return true;
  atomicAdd(&g_bounds_hits, 1);
  g_bounds_last[0] = i;
  g_bounds_last[1] = line;
  return false;
}
#define BONES_INDEX_OK(idx, lo, hi) bones::bones_index_ok((long long)(idx), (long long)(lo), (long long)(hi), __LINE__)
// one per source file: reads and clears that file's counter; last[0] = the offending index, last[1] = the source line
#define BONES_BOUNDS_EXPORT(tu)                                                    \
  extern "C" int bones_bounds_hits_##tu(long long* last) {                          \
    int h = 0, z = 0;                                                               \
    if (cudaMemcpyFromSymbol(&h, bones::g_bounds_hits, sizeof(int)) != cudaSuccess) return -1;   \
    if (last) cudaMemcpyFromSymbol(last, bones::g_bounds_last, 2 * sizeof(long long));           \
    cudaMemcpyToSymbol(bones::g_bounds_hits, &z, sizeof(int));                      \
    return h;                                                                       \
  }
#else
#define BONES_INDEX_OK(idx, lo, hi) true
#define BONES_BOUNDS_EXPORT(tu)
#endif

}  // namespace bones

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
#define BONES_CHECK(x)                                                         \
  do {                                                                         \
    cudaError_t e_ = (x);                                                      \
    if (e_ != cudaSuccess) return (int)e_;                                     \
  } while (0)

namespace bones {
// cuTensorMapEncodeTiled resolved at run time so the library needs no link-time dependency on the driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();
int* error_word();             // device pointer to the library's error word (allocated on first use per device)
int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims, const uint64_t* strides_bytes,
              const uint32_t* box, CUtensorMapSwizzle swz);
}  // namespace bones
