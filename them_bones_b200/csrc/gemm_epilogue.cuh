// Epilogue shared by the bf16 GEMM kernels: one thread turns 32 consecutive accumulator columns of its row into output.
// Every loop over the 32 values is fully unrolled with compile-time indices, including the ragged right edge (handled
// by predication), so the values stay in registers on every path.
#pragma once
#include "common.cuh"

namespace bones {

enum GemmEpi : int { GE_BF16 = 0, GE_BF16_RES = 1, GE_RELU2 = 2, GE_ACC_F32 = 3, GE_MUL_2SQRT = 4, GE_F32 = 5, GE_F32_RES = 6,
                     GE_SOFTCAP = 7 };   // D(bf16) = beta * tanh(alpha * acc): logit soft-capping with alpha = 1 / cap, beta = cap

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sqrt_fast(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// acc      32 fp32 accumulator values (raw bits) of columns [col0, col0 + 32) of this thread's row
// D, R     first element of that span in the output / auxiliary operand (bf16 or fp32 according to `epi`)
// ncols    valid columns in the span (1..32)
// wide     the span starts on a 32-byte boundary in D (and R): 256-bit accesses
// atomic   GE_ACC_F32 only: add with vector atomics (split-K partial tiles)
// pre      GE_BF16_RES / GE_MUL_2SQRT with have_pre: the 32 bf16 of R fetched earlier
__device__ __forceinline__ void gemm_store_chunk(const uint32_t (&acc)[32], int epi, float alpha, float beta, bool wide, bool atomic, void* Dv,
                                                 const void* Rv, bool have_pre, const uint4 (&pre)[4], int ncols) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]) * alpha;
  const bool full = ncols >= 32;
  if (epi == GE_BF16 || epi == GE_BF16_RES || epi == GE_RELU2 || epi == GE_MUL_2SQRT || epi == GE_SOFTCAP) {
    __nv_bfloat16* D = reinterpret_cast<__nv_bfloat16*>(Dv);
    const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(Rv);
    if (epi == GE_BF16_RES || epi == GE_MUL_2SQRT) {
      float f[32];
      if (full) {
        uint4 rr[4];
        if (have_pre) {
#pragma unroll
          for (int j = 0; j < 4; ++j) rr[j] = pre[j];
        } else if (wide) {
          ld_global_v8(R, rr[0], rr[1]);
          ld_global_v8(R + 16, rr[2], rr[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) rr[j] = *reinterpret_cast<const uint4*>(R + j * 8);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 a = unpack_bf16(rr[j].x), b = unpack_bf16(rr[j].y), c = unpack_bf16(rr[j].z), d = unpack_bf16(rr[j].w);
          f[j * 8 + 0] = a.x; f[j * 8 + 1] = a.y; f[j * 8 + 2] = b.x; f[j * 8 + 3] = b.y;
          f[j * 8 + 4] = c.x; f[j * 8 + 5] = c.y; f[j * 8 + 6] = d.x; f[j * 8 + 7] = d.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = j < ncols ? __bfloat162float(R[j]) : 0.f;
      }
      if (epi == GE_BF16_RES) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaf(beta, f[j], v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= 2.0f * sqrt_fast(f[j]);
      }
    } else if (epi == GE_RELU2) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float t = fmaxf(v[j], 0.0f);
        v[j] = t * t;
      }
    } else if (epi == GE_SOFTCAP) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = beta * tanh_approx(v[j]);
    }
    if (full) {
      uint4 uu[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uu[j].x = pack_bf16(v[j * 8 + 0], v[j * 8 + 1]);
        uu[j].y = pack_bf16(v[j * 8 + 2], v[j * 8 + 3]);
        uu[j].z = pack_bf16(v[j * 8 + 4], v[j * 8 + 5]);
        uu[j].w = pack_bf16(v[j * 8 + 6], v[j * 8 + 7]);
      }
      if (wide) {            // one full 32-byte sector per store
        st_global_v8(D, uu[0], uu[1]);
        st_global_v8(D + 16, uu[2], uu[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(D + j * 8) = uu[j];
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) D[j] = __float2bfloat16(v[j]);
    }
    return;
  }
  float* D = reinterpret_cast<float*>(Dv);
  const float* R = reinterpret_cast<const float*>(Rv);
  if (full) {
    if (epi == GE_ACC_F32 && atomic) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(reinterpret_cast<float4*>(D + 4 * j), make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
      return;
    }
    const float* S = epi == GE_ACC_F32 ? D : R;
    const float sc = epi == GE_ACC_F32 ? 1.0f : beta;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (epi != GE_F32) {
        uint4 a, b;
        if (wide) {
          ld_global_v8(S + 8 * g, a, b);
        } else {
          a = *reinterpret_cast<const uint4*>(S + 8 * g);
          b = *reinterpret_cast<const uint4*>(S + 8 * g + 4);
        }
        v[8 * g + 0] = fmaf(sc, __uint_as_float(a.x), v[8 * g + 0]); v[8 * g + 1] = fmaf(sc, __uint_as_float(a.y), v[8 * g + 1]);
        v[8 * g + 2] = fmaf(sc, __uint_as_float(a.z), v[8 * g + 2]); v[8 * g + 3] = fmaf(sc, __uint_as_float(a.w), v[8 * g + 3]);
        v[8 * g + 4] = fmaf(sc, __uint_as_float(b.x), v[8 * g + 4]); v[8 * g + 5] = fmaf(sc, __uint_as_float(b.y), v[8 * g + 5]);
        v[8 * g + 6] = fmaf(sc, __uint_as_float(b.z), v[8 * g + 6]); v[8 * g + 7] = fmaf(sc, __uint_as_float(b.w), v[8 * g + 7]);
      }
      const uint4 o0 = make_uint4(__float_as_uint(v[8 * g + 0]), __float_as_uint(v[8 * g + 1]), __float_as_uint(v[8 * g + 2]),
                                  __float_as_uint(v[8 * g + 3]));
      const uint4 o1 = make_uint4(__float_as_uint(v[8 * g + 4]), __float_as_uint(v[8 * g + 5]), __float_as_uint(v[8 * g + 6]),
                                  __float_as_uint(v[8 * g + 7]));
      if (wide) {
        st_global_v8(D + 8 * g, o0, o1);
      } else {
        *reinterpret_cast<uint4*>(D + 8 * g) = o0;
        *reinterpret_cast<uint4*>(D + 8 * g + 4) = o1;
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (j < ncols) {
      if (epi == GE_ACC_F32 && atomic) {
        atomicAdd(D + j, v[j]);
      } else {
        float x = v[j];
        if (epi == GE_ACC_F32) x += D[j];
        else if (epi == GE_F32_RES) x = fmaf(beta, R[j], x);
        D[j] = x;
      }
    }
  }
}

}  // namespace bones
