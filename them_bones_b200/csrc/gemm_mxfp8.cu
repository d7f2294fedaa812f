// MXFP8 block-scaled GEMM on tcgen05 (`kind::mxf8f6f4.block_scale`) and the quantiser that feeds it.
//
//   D[M,N] = epilogue( (A_q * 2^sfa)[M,K] * (B_q * 2^sfb)[N,K]^T , R )
// A_q, B_q: E4M3 elements, K-major.  Scales: one UE8M0 byte per 1 x 32 block along K (OCP microscaling).  The tensor
// core applies both operands' scales itself; the scale bytes sit in TMEM next to the accumulators, copied there from
// shared memory by `tcgen05.cp` right before the MMAs of each K block.
//
// Scale layout in global memory (chosen so no shuffle is ever needed): for 128-row group g and 128-column K block kb one
// 512-byte chunk at ((g * KB + kb) * 512); inside it byte (r % 32) * 16 + ((r % 128) / 32) * 4 + ((k % 128) / 32).  That
// is exactly the 32-lane x 128-bit image `tcgen05.cp.32x128b.warpx4` spreads over four TMEM columns: lane r % 32, column
// (r % 128) / 32, byte = K sub-block, which the instruction descriptor's scale ids select.
//
// Tile 128 x 160 (N = 160 keeps two accumulators plus the scale columns inside the 512 TMEM columns and divides 1280,
// 3840 and 5120), K block 128, 5 TMA stages.  Warp roles as in gemm_bf16.cu.  Epilogues: bf16 store, residual add,
// ReLU^2, ReLU^2 backward (acc * 2 sqrt(h)), each optionally also emitting the result re-quantised to MXFP8 along N:
// the epilogue thread owns one row and 32 consecutive columns = one scale block of the *next* GEMM's K axis, so the
// fused c_fc -> ReLU^2 -> c_proj chain never re-reads the bf16 activations to quantise them.
//
// Reference counterparts: fp8 fused MLP (round2/source/kernels/nki_mlp_fused8.py:508-570, per-tensor power-of-two
// scales) and fp8 projections (nki_attn_tt8g.py); here per-block scales replace the per-tensor scale statistics.
#include "common.cuh"

namespace bones {

enum MxEpi : int { MX_BF16 = 0, MX_BF16_RES = 1, MX_RELU2 = 2, MX_MUL_2SQRT = 4 };

struct MxParams {
  int M, N, K;
  int epi;
  float beta;
  __nv_bfloat16* D;
  long long ldd;
  const __nv_bfloat16* R;
  long long ldr;
  const uint8_t* sfa;   // scale chunks of A: [ceil(M/128)][K/128][512]
  const uint8_t* sfb;   // scale chunks of B: [ceil(N/160)][K/128][2][512]
  uint8_t* Dq;          // optional: quantised output [M, N] (E4M3)
  uint8_t* Dsf;         // optional: its scales [ceil(M/128)][N/128][512]
  int* err;
  int tiles_m, tiles_n;
};

constexpr int XM = 128, XN = 160, XK = 128, XSTAGES = 5;
constexpr uint32_t XA_BYTES = XM * XK;          // 16384
constexpr uint32_t XB_BYTES = XN * XK;          // 20480
constexpr uint32_t XSFA_BYTES = 512, XSFB_BYTES = 1024;
constexpr uint32_t XSTAGE_BYTES = XA_BYTES + XB_BYTES + XSFA_BYTES + XSFB_BYTES;   // 38400 (a multiple of 1024: 37.5 KB)
constexpr uint32_t XSTAGE_STRIDE = 38912;       // padded to a multiple of 1024 so every stage's tiles stay 1024-aligned
constexpr uint32_t XTMEM_SFA = 320, XTMEM_SFB = 324;

__device__ __forceinline__ float e4m3_scale_pow2(float amax, int& biased) {
  // smallest power of two 2^e with amax / 2^e <= 448 = 1.75 * 2^8
  if (!(amax > 0.f)) { biased = 0; return 0.f; }
  const uint32_t bits = __float_as_uint(amax);
  int e = (int)((bits >> 23) & 0xff) - 127 - 8;
  if ((bits & 0x7fffffu) > 0x600000u) e += 1;      // mantissa above 1.75
  e = max(-127, min(127, e));
  biased = e + 127;
  return __uint_as_float((uint32_t)(127 - e) << 23);   // 2^-e (exact), e in [-127, 127] -> exponent field 0..254
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// `group` is the row-group size of the operand's role: 128 for an A operand (one chunk per group), 160 for a B operand
// (the N tile; two chunks per group, the second holding rows 128..159) so that every tile's scales start at an aligned
// TMEM column.
__device__ __forceinline__ size_t sf_offset(long long r, long long k, long long kblocks, int group) {
  const long long g = r / group, t = r - g * group;
  const int chunks = (group + 127) >> 7;
  return (size_t)(((g * kblocks + (k >> 7)) * chunks + (t >> 7)) * 512 + (t & 31) * 16 + ((t & 127) >> 5) * 4 + ((k & 127) >> 5));
}

// Row quantiser: x bf16 [R, K] -> q E4M3 [R, K] + scale chunks.  One thread per 1 x 32 block.  With `relu2` the input
// is replaced by relu(x)^2 first.
__global__ void mx_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
                                     uint8_t* __restrict__ sf, long long R, long long K, int group) {
  const long long blocks_per_row = K >> 5;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= R * blocks_per_row) return;
  const long long r = i / blocks_per_row, kb = i - r * blocks_per_row;
  const __nv_bfloat16* src = x + r * ldx + kb * 32;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 u = *reinterpret_cast<const uint4*>(src + j * 8);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 f = unpack_bf16(w[t]);
      v[j * 8 + 2 * t] = f.x;
      v[j * 8 + 2 * t + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  int biased;
  const float inv = e4m3_scale_pow2(amax, biased);
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = pack_e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
  uint8_t* dst = q + r * ldq + kb * 32;
  *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<uint4*>(dst + 16) = make_uint4(o[4], o[5], o[6], o[7]);
  sf[sf_offset(r, kb * 32, K >> 7, group)] = (uint8_t)biased;
}

__global__ void __launch_bounds__(192, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t bars = base + XSTAGES * XSTAGE_STRIDE;
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (XSTAGES + s); };
  auto tfull = [&](int a) { return bars + 8u * (2 * XSTAGES + a); };
  auto tempty = [&](int a) { return bars + 8u * (2 * XSTAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * XSTAGES + 4);
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + XSTAGES * XSTAGE_STRIDE + 8 * (2 * XSTAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + XSTAGES * XSTAGE_STRIDE + 8 * (2 * XSTAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < XSTAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull(a), 1);
      mbar_init(tempty(a), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_g;

  const int total = p.tiles_m * p.tiles_n;
  const int KB = p.K / XK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int mb = tile % p.tiles_m, nb = tile / p.tiles_m;
        const int n0 = nb * XN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_arrive_expect_tx(full(stage), XSTAGE_BYTES);
          const uint32_t sa = base + stage * XSTAGE_STRIDE, sb = sa + XA_BYTES, ssfa = sb + XB_BYTES, ssfb = ssfa + XSFA_BYTES;
          tma_load_2d(sa, &tma_a, full(stage), kb * XK, mb * XM);
          tma_load_2d(sb, &tma_b, full(stage), kb * XK, n0);
          bulk_load(ssfa, p.sfa + ((size_t)mb * KB + kb) * 512, 512, full(stage));
          bulk_load(ssfb, p.sfb + ((size_t)nb * KB + kb) * 1024, 1024, full(stage));
          if (++stage == XSTAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const uint32_t sfb_col = XTMEM_SFB;      // the B operand's scales are stored per 160-row tile: always column-aligned
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * XN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(full(stage), phase, abort_flag, p.err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * XSTAGE_STRIDE, sb = sa + XA_BYTES, ssfa = sb + XB_BYTES, ssfb = ssfa + XSFA_BYTES;
          tc_cp_32x128b_warpx4(tmem + XTMEM_SFA, umma_smem_desc(ssfa, 0, 128, kLayoutNone));
          tc_cp_32x128b_warpx4(tmem + XTMEM_SFB, umma_smem_desc(ssfb, 0, 128, kLayoutNone));
          tc_cp_32x128b_warpx4(tmem + XTMEM_SFB + 4, umma_smem_desc(ssfb + 512, 0, 128, kLayoutNone));
          const uint64_t adesc = umma_smem_desc(sa, 0, 1024, kLayoutSw128);
          const uint64_t bdesc = umma_smem_desc(sb, 0, 1024, kLayoutSw128);
#pragma unroll
          for (int k = 0; k < XK / 32; ++k) {
            const uint32_t idesc = umma_idesc_mxf8(XM, XN, 0, 0, 0, 0, (uint32_t)k, (uint32_t)k);
            umma_mxf8(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u, tmem + XTMEM_SFA,
                      tmem + sfb_col);
          }
          tc_commit(empty(stage));
          if (++stage == XSTAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const long long nblocks128 = (p.N + 127) >> 7;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      const int mb = tile % p.tiles_m, nb = tile / p.tiles_m;
      const bool got = mbar_wait(tfull(acc), acc_phase, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const int row = mb * XM + q * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < XN / 32; ++c) {
        uint32_t r[32];
        __syncwarp();
        BONES_TMEM_LD32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * XN + c * 32), r);
        tmem_ld_wait();
        const int col0 = nb * XN + c * 32;
        if (row_ok && col0 + 32 <= p.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (p.epi == MX_BF16_RES || p.epi == MX_MUL_2SQRT) {
            const __nv_bfloat16* R = p.R + (long long)row * p.ldr + col0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 u = *reinterpret_cast<const uint4*>(R + j * 8);
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const float2 f = unpack_bf16(w[t]);
                if (p.epi == MX_BF16_RES) {
                  v[j * 8 + 2 * t] += p.beta * f.x;
                  v[j * 8 + 2 * t + 1] += p.beta * f.y;
                } else {
                  v[j * 8 + 2 * t] *= 2.0f * sqrtf(f.x);
                  v[j * 8 + 2 * t + 1] *= 2.0f * sqrtf(f.y);
                }
              }
            }
          } else if (p.epi == MX_RELU2) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float t = fmaxf(v[j], 0.0f);
              v[j] = t * t;
            }
          }
          __nv_bfloat16* D = p.D + (long long)row * p.ldd + col0;
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 u;
            u.x = pack_bf16(v[j * 8 + 0], v[j * 8 + 1]);
            u.y = pack_bf16(v[j * 8 + 2], v[j * 8 + 3]);
            u.z = pack_bf16(v[j * 8 + 4], v[j * 8 + 5]);
            u.w = pack_bf16(v[j * 8 + 6], v[j * 8 + 7]);
            *reinterpret_cast<uint4*>(D + j * 8) = u;
            if (p.Dq) {
              // quantise what was stored (the bf16-rounded values) so both copies describe the same tensor
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const float2 f = unpack_bf16(w[t]);
                v[j * 8 + 2 * t] = f.x;
                v[j * 8 + 2 * t + 1] = f.y;
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
              }
            }
          }
          if (p.Dq) {
            int biased;
            const float inv = e4m3_scale_pow2(amax, biased);
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = pack_e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
            uint8_t* dq = p.Dq + (long long)row * p.N + col0;
            *reinterpret_cast<uint4*>(dq) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dq + 16) = make_uint4(o[4], o[5], o[6], o[7]);
            p.Dsf[sf_offset(row, col0, nblocks128, 128)] = (uint8_t)biased;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

static int tmap_fp8(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
  uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)ld};
  uint32_t box[2] = {XK, (uint32_t)box_rows};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace bones

extern "C" {
using namespace bones;

// Bytes needed for the scale chunks of an operand with `rows` rows and K columns in row groups of `group` (128: A
// operand, 160: B operand).
long long bones_mx_sf_bytes(long long rows, long long K, int group) {
  return ((rows + group - 1) / group) * (K >> 7) * ((group + 127) >> 7) * 512;
}

int bones_mx_quant_rows(const void* x, long long ldx, void* q, long long ldq, void* sf, long long R, long long K, int group, void* stream) {
  if ((K % 128) || (ldx % 8) || (ldq % 16) || (group != 128 && group != 160)) return -2;
  const long long n = R * (K >> 5);
  mx_quant_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, (uint8_t*)sf, R, K, group);
  return (int)cudaGetLastError();
}

// A_q [M, K] / B_q [N, K] E4M3 row-major (ld = K); D bf16 [M, N]; optional Dq/Dsf: the output re-quantised along N.
int bones_gemm_mxfp8(const void* Aq, const void* sfa, const void* Bq, const void* sfb, void* D, const void* R, void* Dq, void* Dsf, int M,
                     int N, int K, long long ldd, long long ldr, int epi, float beta, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 128) || (N % 32) || (ldd % 8) || ((uintptr_t)Aq & 15) || ((uintptr_t)Bq & 15)) return -2;
  if (Dq && (N % 128)) return -3;
  MxParams p;
  p.M = M; p.N = N; p.K = K; p.epi = epi; p.beta = beta;
  p.D = (__nv_bfloat16*)D; p.ldd = ldd;
  p.R = (const __nv_bfloat16*)(R ? R : D); p.ldr = R ? ldr : ldd;
  p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb;
  p.Dq = (uint8_t*)Dq; p.Dsf = (uint8_t*)Dsf;
  p.err = error_word();
  p.tiles_m = (M + XM - 1) / XM;
  p.tiles_n = (N + XN - 1) / XN;
  CUtensorMap ta, tb;
  int rc = tmap_fp8(&ta, Aq, M, K, K, XM);
  if (rc) return rc;
  rc = tmap_fp8(&tb, Bq, N, K, K, XN);
  if (rc) return rc;
  constexpr size_t smem = (size_t)XSTAGES * XSTAGE_STRIDE + 8 * (2 * XSTAGES + 4) + 16 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int total = p.tiles_m * p.tiles_n;
  gemm_mxfp8_kernel<<<total < sms ? total : sms, 192, smem, (cudaStream_t)stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}
}  // extern "C"
