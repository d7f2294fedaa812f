// Single-token decoding with a KV cache (head_dim 128): the two kernels between the projections of one decode step.
// Both read the current position from device memory, so a whole decode step can be captured once in a CUDA graph and
// replayed for every generated token.
//
//   decode_qkv_kernel    RoPE + QK-norm of the new token's q and k, value-embedding add on v; q goes to a scratch
//                        buffer, k and v are appended to the cache at the current position
//   acc_finish_kernel    tail of the split-K projections of a decode step (few rows, so the contraction is split over
//                        the SMs to stream the weights at memory speed): ordered sum of the fp32 slices -> bf16,
//                        ReLU^2 or residual
//   decode_attn_kernel   one CTA per (head, sequence): soft-max of q . K over the cached keys of the current document
//                        (and window), weighted sum of V.  The fixed soft-max shift of the forward kernel applies
//                        (q and k are RMS-normalised), so no running maximum is kept.
// The reference scores teacher-forced sequences only (round2/submission/inference.py:26-27); decoding is an addition.
#include "common.cuh"

namespace bones {

constexpr float kDecEps = 1.1920928955078125e-07f;   // 2^-23, as in the training kernels

// cache layout: [B, Tmax, H, 128] bf16 (one layer); qkv: [B, 3*H*128]; qbuf: [B, H*128]
__global__ void decode_qkv_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT, const float* __restrict__ sinT,
                                  const __nv_bfloat16* __restrict__ ve, const float* __restrict__ ve_lambda,
                                  __nv_bfloat16* __restrict__ qbuf, __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                                  const int* __restrict__ pos_ptr, int B, int H, int Tmax) {
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);      // (sequence, q|k|v, head)
  const int lane = threadIdx.x & 31;
  if (item >= B * 3 * H) return;
  const int h = item % H, which = (item / H) % 3, b = item / (3 * H);
  const int pos = *pos_ptr;
  if (pos < 0 || pos >= Tmax) return;
  const long long A = (long long)H * 128;
  const __nv_bfloat16* src = qkv + (long long)b * 3 * A + which * A + (long long)h * 128;
  const long long crow = (((long long)b * Tmax + pos) * H + h) * 128;
  // lane owns dims 2*lane, 2*lane+1 of the first half and the same two of the second half (the RoPE partners)
  const float2 x1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + 2 * lane));
  const float2 x2 = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + 64 + 2 * lane));
  if (which == 2) {
    float2 v1 = x1, v2 = x2;
    if (ve) {
      const float g = __bfloat162float(__float2bfloat16(*ve_lambda));   // the gain is applied in bf16, as in training
      const __nv_bfloat16* e = ve + (long long)b * A + (long long)h * 128;
      const float2 e1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(e + 2 * lane));
      const float2 e2 = unpack_bf16(*reinterpret_cast<const uint32_t*>(e + 64 + 2 * lane));
      // the training path rounds v and the scaled embedding to bf16 before adding them
      v1.x = x1.x + __bfloat162float(__float2bfloat16(g * e1.x)); v1.y = x1.y + __bfloat162float(__float2bfloat16(g * e1.y));
      v2.x = x2.x + __bfloat162float(__float2bfloat16(g * e2.x)); v2.y = x2.y + __bfloat162float(__float2bfloat16(g * e2.y));
    }
    *reinterpret_cast<uint32_t*>(vcache + crow + 2 * lane) = pack_bf16(v1.x, v1.y);
    *reinterpret_cast<uint32_t*>(vcache + crow + 64 + 2 * lane) = pack_bf16(v2.x, v2.y);
    return;
  }
  const float2 cs = *reinterpret_cast<const float2*>(cosT + (long long)pos * 64 + 2 * lane);
  const float2 sn = *reinterpret_cast<const float2*>(sinT + (long long)pos * 64 + 2 * lane);
  float2 y1, y2;
  y1.x = x1.x * cs.x + x2.x * sn.x; y1.y = x1.y * cs.y + x2.y * sn.y;
  y2.x = -x1.x * sn.x + x2.x * cs.x; y2.y = -x1.y * sn.y + x2.y * cs.y;
  float ss = y1.x * y1.x + y1.y * y1.y + y2.x * y2.x + y2.y * y2.y;
  ss = warp_sum(ss);
  const float r = rsqrtf(ss * (1.0f / 128.0f) + kDecEps);
  __nv_bfloat16* dst = which == 0 ? qbuf + (long long)b * A + (long long)h * 128 : kcache + crow;
  *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16(y1.x * r, y1.y * r);
  *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16(y2.x * r, y2.y * r);
}

// y[b, h*128 + d] = sum_j softmax_j(scale * q . k_j) v_j over keys lo(b) <= j <= pos.
// Eight lanes share a key (16 dims each), so a warp handles four keys per step and a CTA of eight warps 32.
__global__ void __launch_bounds__(256) decode_attn_kernel(const __nv_bfloat16* __restrict__ qbuf, const __nv_bfloat16* __restrict__ kcache,
                                                          const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ pos_ptr,
                                                          const int* __restrict__ doc_start, __nv_bfloat16* __restrict__ y, int H, int Tmax,
                                                          float scale, int window_tiles) {
  const int h = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, l8 = lane & 7;
  const int pos = *pos_ptr;
  __shared__ float s_acc[8][128];
  __shared__ float s_l[8];
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  float l = 0.f;
  if (pos >= 0 && pos < Tmax) {
    int lo = doc_start ? doc_start[b] : 0;
    if (window_tiles > 0) lo = max(lo, (pos / 128 - (window_tiles - 1)) * 128);
    lo = max(lo, 0);
    const long long A = (long long)H * 128;
    float q[16];
    {
      const __nv_bfloat16* qp = qbuf + (long long)b * A + (long long)h * 128 + l8 * 16;
      const uint4 u0 = *reinterpret_cast<const uint4*>(qp), u1 = *reinterpret_cast<const uint4*>(qp + 8);
      const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = unpack_bf16(w[i]);
        q[2 * i] = f.x; q[2 * i + 1] = f.y;
      }
    }
    const float c1 = scale * 1.4426950408889634f, c2 = scale * 128.0f * 1.4426950408889634f;
    for (int j0 = lo + warp * 4; j0 <= pos; j0 += 32) {
      const int j = j0 + grp;
      const bool live = j <= pos;
      const long long off = (((long long)b * Tmax + (live ? j : pos)) * H + h) * 128 + l8 * 16;
      const uint4 k0 = *reinterpret_cast<const uint4*>(kcache + off), k1 = *reinterpret_cast<const uint4*>(kcache + off + 8);
      const uint4 v0 = *reinterpret_cast<const uint4*>(vcache + off), v1 = *reinterpret_cast<const uint4*>(vcache + off + 8);
      const uint32_t kw[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = unpack_bf16(kw[i]);
        s += q[2 * i] * f.x + q[2 * i + 1] * f.y;
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      const float p = live ? exp2f(s * c1 - c2) : 0.f;
      l += p;
      const uint32_t vw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = unpack_bf16(vw[i]);
        acc[2 * i] += p * f.x; acc[2 * i + 1] += p * f.y;
      }
    }
  }
  // the four key groups of a warp hold partial sums for the same 16 dims per l8: fold them, then fold the warps
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
    acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
  }
  l += __shfl_xor_sync(0xffffffffu, l, 8);
  l += __shfl_xor_sync(0xffffffffu, l, 16);
  if (grp == 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i) s_acc[warp][l8 * 16 + i] = acc[i];
    if (l8 == 0) s_l[warp] = l;
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    float o = 0.f, lt = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { o += s_acc[w][threadIdx.x]; lt += s_l[w]; }
    y[((long long)b * H + h) * 128 + threadIdx.x] = __float2bfloat16(lt > 0.f ? o / lt : 0.f);
  }
}

// Tail of a split-K decode projection: the GEMM ran as `splits` batched products over K chunks, each writing its own fp32
// slice; the slices are added in a fixed order (so a decode step is reproducible bit for bit) and become the bf16
// output, optionally through ReLU^2 (mode 2) or plus a bf16 residual (mode 1).
__global__ void acc_finish_kernel(const float* __restrict__ part, int splits, long long slice, const __nv_bfloat16* __restrict__ residual,
                                  __nv_bfloat16* __restrict__ out, long long n, int mode) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 v = *reinterpret_cast<const float4*>(part + i);
  for (int s = 1; s < splits; ++s) {
    const float4 u = *reinterpret_cast<const float4*>(part + (long long)s * slice + i);
    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
  }
  if (mode == 2) {
    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
    v.x *= v.x; v.y *= v.y; v.z *= v.z; v.w *= v.w;
  } else if (mode == 1) {
    const uint2 r = *reinterpret_cast<const uint2*>(residual + i);
    const float2 r0 = unpack_bf16(r.x), r1 = unpack_bf16(r.y);
    v.x += r0.x; v.y += r0.y; v.z += r1.x; v.w += r1.y;
  }
  *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

}  // namespace bones

extern "C" {
using namespace bones;

int bones_acc_finish(const float* part, int splits, long long slice, const void* residual, void* out, long long n, int mode, void* stream) {
  if (n % 4 || slice % 4 || splits < 1 || (mode == 1 && !residual)) return -2;
  if (n == 0) return 0;
  acc_finish_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(part, splits, slice, (const __nv_bfloat16*)residual,
                                                                                      (__nv_bfloat16*)out, n, mode);
  return (int)cudaGetLastError();
}

int bones_decode_qkv(const void* qkv, const float* cosT, const float* sinT, const void* ve, const float* ve_lambda, void* qbuf, void* kcache,
                     void* vcache, const int* pos, int B, int H, int Tmax, void* stream) {
  const int warps = B * 3 * H;
  decode_qkv_kernel<<<(warps + 7) / 8, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)qkv, cosT, sinT, (const __nv_bfloat16*)ve,
                                                                       ve_lambda, (__nv_bfloat16*)qbuf, (__nv_bfloat16*)kcache,
                                                                       (__nv_bfloat16*)vcache, pos, B, H, Tmax);
  return (int)cudaGetLastError();
}

int bones_decode_attn(const void* qbuf, const void* kcache, const void* vcache, const int* pos, const int* doc_start, void* y, int B, int H,
                      int Tmax, float scale, int window_tiles, void* stream) {
  dim3 grid(H, B);
  decode_attn_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)qbuf, (const __nv_bfloat16*)kcache,
                                                             (const __nv_bfloat16*)vcache, pos, doc_start, (__nv_bfloat16*)y, H, Tmax, scale,
                                                             window_tiles);
  return (int)cudaGetLastError();
}
}  // extern "C"
