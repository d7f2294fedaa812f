// The element-wise tail of a Muon step after Newton-Schulz, on stacks [k, r, c] of one shape group
// (reference: the NorMuon second-moment rescale, cautious weight decay and master update of ``_muon_math``,
// round2/source/train.py:12882; PyTorch statement: ref/functional.py::muon_update):
//
//   muon_linesq_rows / _cols   v[line] = mean over the reduced dimension of g^2 (rows of a tall matrix, columns of a wide one)
//   muon_apply                 w -= lr * (g * s[line]) + lr * wd * w * [g * s[line] * w >= 0]
//
// The per-line arithmetic between the two (second-moment update, step size, norm-preserving ratio) works on k * r or
// k * c values and stays in PyTorch.  One read of g for the statistics, one read of g and one read-modify-write of the
// fp32 master for the update.
#include "common.cuh"

namespace bones {

// one warp per line of c elements (c even)
__global__ void muon_linesq_rows_kernel(const __nv_bfloat16* __restrict__ g, float* __restrict__ out, long long lines, int c) {
  const long long line = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (line >= lines) return;
  const __nv_bfloat16* p = g + line * c;
  float s = 0.f;
  for (int j = lane * 2; j < c; j += 64) {
    const float2 f = unpack_bf16(*reinterpret_cast<const uint32_t*>(p + j));
    s += f.x * f.x + f.y * f.y;
  }
  s = warp_sum(s);
  if (lane == 0) out[line] = s / (float)c;
}

// grid (ceil(c / 2 / 256), segments, k); each thread owns two adjacent columns over its segment of rows; out is zeroed
__global__ void muon_linesq_cols_kernel(const __nv_bfloat16* __restrict__ g, float* __restrict__ out, int r, int c, int rows_per_seg) {
  const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (col >= c) return;
  const int k = blockIdx.z;
  const int r0 = blockIdx.y * rows_per_seg, r1 = min(r, r0 + rows_per_seg);
  const __nv_bfloat16* p = g + ((long long)k * r + r0) * c + col;
  float s0 = 0.f, s1 = 0.f;
  for (int i = r0; i < r1; ++i, p += c) {
    const float2 f = unpack_bf16(*reinterpret_cast<const uint32_t*>(p));
    s0 += f.x * f.x;
    s1 += f.y * f.y;
  }
  const float inv = 1.0f / (float)r;
  atomicAdd(out + (long long)k * c + col, s0 * inv);
  atomicAdd(out + (long long)k * c + col + 1, s1 * inv);
}

// two elements per thread (c even, so a pair never straddles a row)
__global__ void muon_apply_kernel(const __nv_bfloat16* __restrict__ g, float* __restrict__ w, const float* __restrict__ line_scale, long long n,
                                  int r, int c, int by_row, float lr, float lr_wd) {
  const long long e = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (e >= n) return;
  const long long mat = (long long)r * c;
  const long long k = e / mat, rem = e - k * mat;
  const int row = (int)(rem / c), col = (int)(rem - (long long)row * c);
  float s0, s1;
  if (by_row) {
    s0 = s1 = line_scale[k * r + row];
  } else {
    s0 = line_scale[k * c + col];
    s1 = line_scale[k * c + col + 1];
  }
  const float2 gv = unpack_bf16(*reinterpret_cast<const uint32_t*>(g + e));
  float2 wv = *reinterpret_cast<const float2*>(w + e);
  const float g0 = gv.x * s0, g1 = gv.y * s1;
  wv.x -= lr * g0 + (g0 * wv.x >= 0.f ? lr_wd * wv.x : 0.f);
  wv.y -= lr * g1 + (g1 * wv.y >= 0.f ? lr_wd * wv.y : 0.f);
  *reinterpret_cast<float2*>(w + e) = wv;
}

}  // namespace bones

extern "C" {
using namespace bones;

// out[k * lines_per_matrix + line]: mean of g^2 along the other dimension.  by_row: one value per row (r >= c).
int bones_muon_linesq(const void* g, float* out, int k, int r, int c, int by_row, void* stream) {
  if (c % 2) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  if (by_row) {
    const long long lines = (long long)k * r;
    muon_linesq_rows_kernel<<<(unsigned)((lines + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)g, out, lines, c);
  } else {
    cudaMemsetAsync(out, 0, sizeof(float) * (size_t)k * c, st);
    const int segs = 8, rows_per_seg = (r + segs - 1) / segs;
    dim3 grid((unsigned)((c / 2 + 255) / 256), segs, k);
    muon_linesq_cols_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, out, r, c, rows_per_seg);
  }
  return (int)cudaGetLastError();
}

int bones_muon_apply(const void* g, float* w, const float* line_scale, int k, int r, int c, int by_row, float lr, float lr_wd, void* stream) {
  if (c % 2) return -2;
  const long long n = (long long)k * r * c;
  muon_apply_kernel<<<(unsigned)((n / 2 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, w, line_scale, n, r, c, by_row, lr,
                                                                                      lr_wd);
  return (int)cudaGetLastError();
}
}  // extern "C"
