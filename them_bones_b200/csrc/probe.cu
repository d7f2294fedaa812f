// Issue-rate probe for tcgen05.mma: one CTA issues a train of 128 x N x 16 bf16 MMAs into one accumulator with the least
// instruction overhead per MMA (descriptor halves precomputed, one add per operand) and times it with clock64.
// Answers how many cycles one such instruction costs against its tensor-pipe time (N / 2 cycles), with the A operand in
// shared memory or in TMEM.  Used by `python -m them_bones_b200.ops.microbench mma`.
#include "common.cuh"

namespace bones {

__global__ void __launch_bounds__(128, 1) mma_probe_kernel(long long* out, int n_mma, int a_tmem, int nsize, int* err) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sA = base, sB = base + 32768, bars = base + 32768 * 3;     // A: 128 x 128, B: 256 x 128 (bf16, SW128)
  volatile uint32_t* slot_g = reinterpret_cast<volatile uint32_t*>(gen + 32768 * 3 + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + 32768 * 3 + 24);
  for (int i = threadIdx.x; i < 32768 * 3 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(gen)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    mbar_init(bars, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  __syncthreads();
  if (threadIdx.x < 32) {
    tmem_alloc(bars + 16, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot_g;
  if (threadIdx.x == 0) {
    const uint32_t idesc = umma_idesc_f16(128, (uint32_t)nsize, 1, 0, 0);
    const uint32_t hi = umma_desc_hi(1024, kLayoutSw128);
    const uint32_t alo = umma_desc_lo(sA, 0), blo = umma_desc_lo(sB, 0);
    const long long t0 = clock64();
    for (int i = 0; i < n_mma; i += 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t off = (uint32_t)(((k >> 2) * 16384 + (k & 3) * 32) >> 4);
        if (a_tmem) umma_f16_ts_lh(tmem, tmem + 384 + (uint32_t)(k * 8), blo + off, hi, idesc, 1u);
        else umma_f16_lh(tmem, alo + off, hi, blo + off, hi, idesc, 1u);
      }
    }
    const long long t1 = clock64();
    tc_commit(bars);
    mbar_wait(bars, 0, abort_flag, err, ERR_WAIT_AUX);
    const long long t2 = clock64();
    out[0] = t1 - t0;
    out[1] = t2 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace bones

extern "C" {
using namespace bones;
// out: two int64 on the device (cycles until the last MMA was issued, cycles until all completed); n_mma a multiple of 8
int bones_mma_probe(long long* out, int n_mma, int a_tmem, int nsize, void* stream) {
  if (n_mma <= 0 || (n_mma % 8) || (nsize != 128 && nsize != 256)) return -2;
  constexpr size_t smem = 32768 * 3 + 64 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  mma_probe_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(out, n_mma, a_tmem, nsize, error_word());
  return (int)cudaGetLastError();
}
}  // extern "C"
