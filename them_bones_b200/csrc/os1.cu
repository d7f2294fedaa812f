// Kernels of the output-side hashed table (a table of sign-hashed rows whose read-out is added to the logits before the
// soft-cap; reference: switch 59, round2/source/train.py:2310-2351).  The two GEMMs of the read-out (scores S = U C^T and
// dU = dLogits C) run on the tensor-core GEMM; these are the element-wise pieces around them:
//
//   os1_signs_kernel     out = signs(hash) * in, the +-1 pattern being the bits of mixed 64-bit words of the hash
//   os1_combine_kernel   logits <- [cap * tanh(. / cap)] (logits + glin * s + gate * k * relu(s - thr)), in place
//   os1_gate_dot_kernel  sd[row] = u[row] . code[next[row]] / a0 (the gate's read of the token that followed)
//   os1_row_step_kernel  the stateless row update: x -= lr g / (rms(g) + eps), then rms(x) <= cap * lr
#include "common.cuh"

namespace bones {

__device__ __forceinline__ unsigned long long os1_mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// one thread per (row, group of 8 columns); dim a multiple of 8
template <typename TI, typename TO>
__global__ void os1_signs_kernel(const TI* __restrict__ in, const long long* __restrict__ hsign, TO* __restrict__ out, long long n, int dim) {
  const int groups = dim >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * groups) return;
  const long long row = i / groups;
  const int c0 = (int)(i % groups) * 8;
  const unsigned long long word = os1_mix64((unsigned long long)hsign[row] + (unsigned long long)(c0 / 64 + 1) * 0x9E3779B97F4A7C15ull);
  const unsigned bits = (unsigned)(word >> (c0 & 63)) & 0xffu;
  const TI* src = in + row * dim + c0;
  TO* dst = out + row * dim + c0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float v = (float)src[j];
    dst[j] = (TO)(((bits >> j) & 1u) ? -v : v);
  }
}

// 8 bf16 per thread; ld = row pitch (elements, a multiple of 8); ncols a multiple of 8
__global__ void os1_combine_kernel(__nv_bfloat16* __restrict__ lg, const __nv_bfloat16* __restrict__ s, const float* __restrict__ gate,
                                   long long rows, int ncols, long long ld, float cap, float glin, float kthr, float thr, int do_cap) {
  const int groups = ncols >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * groups) return;
  const long long row = i / groups;
  const long long off = row * ld + (i % groups) * 8;
  const float g = gate[row] * kthr;
  const uint4 a = *reinterpret_cast<const uint4*>(lg + off);
  const uint4 b = *reinterpret_cast<const uint4*>(s + off);
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t ow[4];
  const float inv = 1.0f / cap;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 x = unpack_bf16(aw[j]), sv = unpack_bf16(bw[j]);
    float y0 = x.x + glin * sv.x + g * fmaxf(sv.x - thr, 0.f);
    float y1 = x.y + glin * sv.y + g * fmaxf(sv.y - thr, 0.f);
    if (do_cap) {
      y0 = cap * tanhf(y0 * inv);
      y1 = cap * tanhf(y1 * inv);
    }
    ow[j] = pack_bf16(y0, y1);
  }
  *reinterpret_cast<uint4*>(lg + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// one warp per row: sd[row] = u[row] . code[next[row]] * inv_a0 (0 where next < 0)
__global__ void os1_gate_dot_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ code, const long long* __restrict__ next,
                                    float* __restrict__ sd, long long n, int dim, float inv_a0) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n) return;
  const long long tk = next[row];
  float acc = 0.f;
  if (tk >= 0) {
    for (int c = lane * 2; c < dim; c += 64) {
      const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(u + row * dim + c));
      const float2 b = unpack_bf16(*reinterpret_cast<const uint32_t*>(code + tk * dim + c));
      acc += a.x * b.x + a.y * b.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) sd[row] = acc * inv_a0;
}

// one warp per touched row; dim <= 256 and a multiple of 32.  T = table element type.
template <typename T>
__global__ void os1_row_step_kernel(T* __restrict__ table, const long long* __restrict__ rows, const float* __restrict__ g, int n, int dim, float lr,
                                    float eps, float cap_lr, int* __restrict__ n_capped) {
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n) return;
  const int per = dim >> 5;
  T* x = table + rows[item] * (long long)dim;
  const float* gr = g + (long long)item * dim;
  float xv[8], gv[8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < per) {
      gv[j] = gr[lane + 32 * j];
      xv[j] = (float)x[lane + 32 * j];
      ss += gv[j] * gv[j];
    }
  }
  ss = warp_sum(ss);
  const float k = lr / (sqrtf(ss / (float)dim) + eps);
  float qq = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < per) {
      xv[j] -= k * gv[j];
      qq += xv[j] * xv[j];
    }
  }
  qq = warp_sum(qq);
  const float f = fminf(cap_lr / fmaxf(sqrtf(qq / (float)dim), 1e-30f), 1.0f);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j < per) x[lane + 32 * j] = (T)(xv[j] * f);
  if (lane == 0 && f < 1.0f && n_capped) atomicAdd(n_capped, 1);
}

}  // namespace bones

extern "C" {
using namespace bones;

// kind 0: bf16 -> bf16 (rows to u), 1: fp32 -> fp32 (dU to row gradients), 2: fp32 -> bf16
int bones_os1_signs(const void* in, const long long* hsign, void* out, long long n, int dim, int kind, void* stream) {
  if (dim % 8) return -1;
  const long long total = n * (dim / 8);
  if (total == 0) return 0;
  const unsigned grid = (unsigned)((total + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == 0) os1_signs_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)in, hsign, (__nv_bfloat16*)out, n, dim);
  else if (kind == 1) os1_signs_kernel<float, float><<<grid, 256, 0, st>>>((const float*)in, hsign, (float*)out, n, dim);
  else os1_signs_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>((const float*)in, hsign, (__nv_bfloat16*)out, n, dim);
  return (int)cudaGetLastError();
}

int bones_os1_combine(void* logits, const void* s, const float* gate, long long rows, int ncols, long long ld, float cap, float glin, float kthr,
                      float thr, int do_cap, void* stream) {
  if (ncols % 8 || ld % 8) return -1;
  const long long total = rows * (ncols / 8);
  if (total == 0) return 0;
  os1_combine_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, (const __nv_bfloat16*)s, gate, rows,
                                                                                      ncols, ld, cap, glin, kthr, thr, do_cap);
  return (int)cudaGetLastError();
}

int bones_os1_gate_dot(const void* u, const void* code, const long long* next, float* sd, long long n, int dim, float inv_a0, void* stream) {
  if (dim % 2) return -1;
  if (n == 0) return 0;
  os1_gate_dot_kernel<<<(unsigned)((n + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)u, (const __nv_bfloat16*)code, next, sd, n, dim,
                                                                                inv_a0);
  return (int)cudaGetLastError();
}

int bones_os1_row_step(void* table, const long long* rows, const float* g, int n, int dim, float lr, float eps, float cap_lr, int* n_capped,
                       int table_is_f32, void* stream) {
  if (dim % 32 || dim > 256) return -1;
  if (n == 0) return 0;
  const unsigned grid = (unsigned)((n + 7) / 8);
  if (table_is_f32) os1_row_step_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((float*)table, rows, g, n, dim, lr, eps, cap_lr, n_capped);
  else os1_row_step_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)table, rows, g, n, dim, lr, eps, cap_lr, n_capped);
  return (int)cudaGetLastError();
}
}  // extern "C"
