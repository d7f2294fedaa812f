// Bandwidth-bound fused blocks: parameter-free RMSNorm, residual mix + norm, embedding gather / scatter-add, softcap
// cross-entropy with in-place logit gradients, row gathers for the MoE slot buffer.
//
// Row kernels use one warp per row with 16-byte vector accesses and keep the row in registers between the reduction and
// the write, so every tensor is read once and written once.  Reductions for scalar-gain gradients are summed per block
// and added with one atomic per block.
//
// Reference counterparts: block head `x' = l1*x + l2*x0; xn = rms(x')` (round1/source/train.py:5257-5301), rms pair
// (:5378-5410), residual-mix backward with gain partial sums (round2/source/kernels/nki_resmix.py), embedding backward
// (round2/source/train.py:5606-5658, there a one-hot contraction), chunked loss head (round2/source/train.py:5238-5297).
#include <cuda_fp16.h>

#include "common.cuh"

namespace bones {

constexpr float kRmsEps = 1.1920928955078125e-07f;   // 2^-23
constexpr int kMaxVec = 8;                           // up to 8 x (32 lanes x 8 bf16) = 2048 columns per row

struct RowRegs {
  float v[kMaxVec][8];
};

__device__ __forceinline__ void load_row(const __nv_bfloat16* row, int C, int lane, RowRegs& r) {
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
      const uint4 u = *reinterpret_cast<const uint4*>(row + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = unpack_bf16(w[t]);
        r.v[i][2 * t] = f.x;
        r.v[i][2 * t + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) r.v[i][t] = 0.f;
    }
  }
}
__device__ __forceinline__ void store_row(__nv_bfloat16* row, int C, int lane, const RowRegs& r) {
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * 32 + lane) * 8;
    if (c < C) {
      uint4 u;
      u.x = pack_bf16(r.v[i][0], r.v[i][1]);
      u.y = pack_bf16(r.v[i][2], r.v[i][3]);
      u.z = pack_bf16(r.v[i][4], r.v[i][5]);
      u.w = pack_bf16(r.v[i][6], r.v[i][7]);
      *reinterpret_cast<uint4*>(row + c) = u;
    }
  }
}
__device__ __forceinline__ float row_sumsq(const RowRegs& r) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) s += r.v[i][t] * r.v[i][t];
  return warp_sum(s);
}
__device__ __forceinline__ float row_dot(const RowRegs& a, const RowRegs& b) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) s += a.v[i][t] * b.v[i][t];
  return warp_sum(s);
}

// y = x * rsqrt(mean(x^2) + eps)
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, int M, int C) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  RowRegs r;
  load_row(x + (size_t)row * C, C, lane, r);
  const float rstd = rsqrtf(row_sumsq(r) / C + kRmsEps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) r.v[i][t] *= rstd;
  store_row(y + (size_t)row * C, C, lane, r);
}

// dx = (add ? add : 0) + rstd * (dy - xhat * mean(dy * xhat)),  xhat = x * rstd
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* x, const __nv_bfloat16* dy, const __nv_bfloat16* add, __nv_bfloat16* dx, int M,
                                   int C) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  RowRegs rx, rg;
  load_row(x + (size_t)row * C, C, lane, rx);
  load_row(dy + (size_t)row * C, C, lane, rg);
  const float rstd = rsqrtf(row_sumsq(rx) / C + kRmsEps);
  const float m = row_dot(rx, rg) * rstd * rstd / C;     // mean(dy * xhat) * rstd
  RowRegs ra;
  if (add) load_row(add + (size_t)row * C, C, lane, ra);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      float g = rstd * (rg.v[i][t] - rx.v[i][t] * m);
      if (add) g += ra.v[i][t];
      rg.v[i][t] = g;
    }
  store_row(dx + (size_t)row * C, C, lane, rg);
}

// xm = a*x + b*x0 ; xn = rmsnorm(xm)   (a, b: device scalars)
__global__ void resid_mix_norm_fwd_kernel(const __nv_bfloat16* x, const __nv_bfloat16* x0, const float* a, const float* b,
                                          __nv_bfloat16* xm, __nv_bfloat16* xn, int M, int C) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const float fa = *a, fb = *b;
  RowRegs r, r0;
  load_row(x + (size_t)row * C, C, lane, r);
  load_row(x0 + (size_t)row * C, C, lane, r0);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      // round the mixed stream to bf16 first: the norm sees exactly what is stored
      r.v[i][t] = __bfloat162float(__float2bfloat16(fa * r.v[i][t] + fb * r0.v[i][t]));
    }
  store_row(xm + (size_t)row * C, C, lane, r);
  const float rstd = rsqrtf(row_sumsq(r) / C + kRmsEps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int t = 0; t < 8; ++t) r.v[i][t] *= rstd;
  store_row(xn + (size_t)row * C, C, lane, r);
}

// g = dxm + rmsnorm_bwd(xm, dxn);  dx = a*g;  dx0 = b*g;  da += sum(g*x);  db += sum(g*x0)
__global__ void resid_mix_norm_bwd_kernel(const __nv_bfloat16* x, const __nv_bfloat16* x0, const __nv_bfloat16* xm, const float* a,
                                          const float* b, const __nv_bfloat16* dxm, const __nv_bfloat16* dxn, __nv_bfloat16* dx,
                                          __nv_bfloat16* dx0, float* da, float* db, int M, int C, int acc_x0) {
  __shared__ float s_da[32], s_db[32];
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + wid;
  float pa = 0.f, pb = 0.f;
  if (row < M) {
    const float fa = *a, fb = *b;
    RowRegs rm, rg, rt;
    load_row(xm + (size_t)row * C, C, lane, rm);
    load_row(dxn + (size_t)row * C, C, lane, rg);
    const float rstd = rsqrtf(row_sumsq(rm) / C + kRmsEps);
    const float m = row_dot(rm, rg) * rstd * rstd / C;
    load_row(dxm + (size_t)row * C, C, lane, rt);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
      for (int t = 0; t < 8; ++t) rg.v[i][t] = rt.v[i][t] + rstd * (rg.v[i][t] - rm.v[i][t] * m);
    load_row(x + (size_t)row * C, C, lane, rt);
    pa = row_dot(rg, rt);
    load_row(x0 + (size_t)row * C, C, lane, rt);
    pb = row_dot(rg, rt);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
      for (int t = 0; t < 8; ++t) rt.v[i][t] = fb * rg.v[i][t];
    if (acc_x0) {                       // dx0 accumulates the contributions of all blocks that read x0
      RowRegs ro;
      load_row(dx0 + (size_t)row * C, C, lane, ro);
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
        for (int t = 0; t < 8; ++t) rt.v[i][t] += ro.v[i][t];
    }
    store_row(dx0 + (size_t)row * C, C, lane, rt);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
      for (int t = 0; t < 8; ++t) rg.v[i][t] *= fa;
    store_row(dx + (size_t)row * C, C, lane, rg);
  }
  if (lane == 0) { s_da[wid] = pa; s_db[wid] = pb; }
  __syncthreads();
  if (wid == 0) {
    const int nw = blockDim.x >> 5;
    float va = lane < nw ? s_da[lane] : 0.f, vb = lane < nw ? s_db[lane] : 0.f;
    va = warp_sum(va);
    vb = warp_sum(vb);
    if (lane == 0) { atomicAdd(da, va); atomicAdd(db, vb); }
  }
}

// Row kernels for C == NV * 256 that keep every operand packed (one uint4 per 8 columns) and issue all of a row's loads
// before the first reduction: about half the registers of the generic kernels above, so two blocks fit per SM and
// enough loads are in flight to keep DRAM busy.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  return u;
}

template <int NV>
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_packed_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ add,
                          __nv_bfloat16* __restrict__ dx, int M) {
  constexpr int C = NV * 256;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const size_t off = (size_t)row * C + lane * 8;
  uint4 px[NV], pg[NV], pa[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) px[i] = *reinterpret_cast<const uint4*>(x + off + i * 256);
#pragma unroll
  for (int i = 0; i < NV; ++i) pg[i] = *reinterpret_cast<const uint4*>(dy + off + i * 256);
  if (add) {
#pragma unroll
    for (int i = 0; i < NV; ++i) pa[i] = *reinterpret_cast<const uint4*>(add + off + i * 256);
  }
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float fx[8], fg[8];
    unpack8(px[i], fx);
    unpack8(pg[i], fg);
#pragma unroll
    for (int t = 0; t < 8; ++t) { ss += fx[t] * fx[t]; dot += fx[t] * fg[t]; }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float rstd = rsqrtf(ss / C + kRmsEps);
  const float m = dot * rstd * rstd / C;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    float fx[8], fg[8], fa[8];
    unpack8(px[i], fx);
    unpack8(pg[i], fg);
    if (add) unpack8(pa[i], fa);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      float g = rstd * (fg[t] - fx[t] * m);
      if (add) g += fa[t];
      fg[t] = g;
    }
    *reinterpret_cast<uint4*>(dx + off + i * 256) = pack8(fg);
  }
}

template <int NV>
__global__ void __launch_bounds__(256, 2)
resid_mix_norm_bwd_packed_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0,
                                 const __nv_bfloat16* __restrict__ xm, const float* __restrict__ a, const float* __restrict__ b,
                                 const __nv_bfloat16* __restrict__ dxm, const __nv_bfloat16* __restrict__ dxn,
                                 __nv_bfloat16* __restrict__ dx, __nv_bfloat16* dx0, float* da, float* db, int M, int acc_x0) {
  constexpr int C = NV * 256;
  __shared__ float s_da[8], s_db[8];
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + wid;
  float pa = 0.f, pb = 0.f;
  if (row < M) {
    const size_t off = (size_t)row * C + lane * 8;
    uint4 pm[NV], pn[NV], pt[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) pm[i] = *reinterpret_cast<const uint4*>(xm + off + i * 256);
#pragma unroll
    for (int i = 0; i < NV; ++i) pn[i] = *reinterpret_cast<const uint4*>(dxn + off + i * 256);
#pragma unroll
    for (int i = 0; i < NV; ++i) pt[i] = *reinterpret_cast<const uint4*>(dxm + off + i * 256);
    const float fa = *a, fb = *b;
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float fm[8], fn[8];
      unpack8(pm[i], fm);
      unpack8(pn[i], fn);
#pragma unroll
      for (int t = 0; t < 8; ++t) { ss += fm[t] * fm[t]; dot += fm[t] * fn[t]; }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rstd = rsqrtf(ss / C + kRmsEps);
    const float m = dot * rstd * rstd / C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      // x and x0 are only needed from here on: fetched per vector, the other warps of the SM cover their latency
      const uint4 px = *reinterpret_cast<const uint4*>(x + off + i * 256);
      const uint4 p0 = *reinterpret_cast<const uint4*>(x0 + off + i * 256);
      float fm[8], fn[8], ft[8], fx[8], f0[8], o[8];
      unpack8(pm[i], fm);
      unpack8(pn[i], fn);
      unpack8(pt[i], ft);
      unpack8(px, fx);
      unpack8(p0, f0);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float g = ft[t] + rstd * (fn[t] - fm[t] * m);
        pa += g * fx[t];
        pb += g * f0[t];
        o[t] = fb * g;
        fn[t] = fa * g;
      }
      if (acc_x0) {                     // dx0 accumulates the contributions of all blocks that read x0
        float old[8];
        unpack8(*reinterpret_cast<const uint4*>(dx0 + off + i * 256), old);
#pragma unroll
        for (int t = 0; t < 8; ++t) o[t] += old[t];
      }
      *reinterpret_cast<uint4*>(dx0 + off + i * 256) = pack8(o);
      *reinterpret_cast<uint4*>(dx + off + i * 256) = pack8(fn);
    }
    pa = warp_sum(pa);
    pb = warp_sum(pb);
  }
  if (lane == 0) { s_da[wid] = pa; s_db[wid] = pb; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float va = 0.f, vb = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { va += s_da[w]; vb += s_db[w]; }
    atomicAdd(da, va);
    atomicAdd(db, vb);
  }
}

// out[i] = table[idx[i]] (bf16 rows); idx == n_rows (the pad id) gives a zero row
template <typename IdxT>
__global__ void gather_rows_kernel(const __nv_bfloat16* table, const IdxT* idx, __nv_bfloat16* out, int n, int C, long long n_rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const long long src = (long long)idx[row];
  (void)BONES_INDEX_OK(src, 0, n_rows + 1);            // n_rows itself is the "empty slot" marker
  const bool valid = src >= 0 && src < n_rows;
  for (int c = lane * 8; c < C; c += 256) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (valid) u = *reinterpret_cast<const uint4*>(table + (size_t)src * C + c);
    *reinterpret_cast<uint4*>(out + (size_t)row * C + c) = u;
  }
}

// grad[idx[i]] += dy[i]  (fp32 accumulation buffer, one vector atomic per 4 columns)
template <typename IdxT>
__global__ void scatter_add_rows_kernel(const __nv_bfloat16* dy, const IdxT* idx, float* grad, int n, int C, long long n_rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const long long dst = (long long)idx[row];
  (void)BONES_INDEX_OK(dst, 0, n_rows + 1);
  if (dst < 0 || dst >= n_rows) return;
  for (int c = lane * 8; c < C; c += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(dy + (size_t)row * C + c);
    const float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z), f3 = unpack_bf16(u.w);
    float4* g = reinterpret_cast<float4*>(grad + (size_t)dst * C + c);
    atomicAdd(g, make_float4(f0.x, f0.y, f1.x, f1.y));
    atomicAdd(g + 1, make_float4(f2.x, f2.y, f3.x, f3.y));
  }
}

// out[n] = sum_k gates[n,k] * ys[slot[n,k]]   (slot == S: dropped)
__global__ void moe_combine_kernel(const __nv_bfloat16* ys, const long long* slot, const float* gates, __nv_bfloat16* out, int n, int C,
                                   int topk, long long S) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  for (int c = lane * 8; c < C; c += 256) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < topk; ++k) {
      const long long s = slot[(size_t)row * topk + k];
      if (s < 0 || s >= S) continue;
      const float g = gates[(size_t)row * topk + k];
      const uint4 u = *reinterpret_cast<const uint4*>(ys + (size_t)s * C + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = unpack_bf16(w[t]);
        acc[2 * t] += g * f.x;
        acc[2 * t + 1] += g * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)row * C + c) = o;
  }
}


// Causal per-sequence capacity slotting (MoE).  One CTA per sequence.  idx [b*t, k] holds each token's expert choices
// (distinct per token).  The position of an assignment is the number of assignments to the same expert at earlier
// tokens of the sequence; positions >= cap are dropped.  Outputs: slot [b*t, k] (index into the [E, b, cap] buffer, or
// E*b*cap when dropped) and tok [E*b*cap] (token in each slot, or b*t when empty).
// Reference semantics: moe_positions / moe_gather_tables (round2/source/train.py:10555-10636), there as tril matmuls.
constexpr int kSlotThreads = 256;
constexpr int kMaxExperts = 64;
__global__ void moe_slots_kernel(const long long* __restrict__ idx, long long* __restrict__ slot, long long* __restrict__ tok, int b, int t,
                                 int k, int n_exp, int cap) {
  __shared__ unsigned short cnt[kMaxExperts][kSlotThreads];
  const int row = blockIdx.x, tid = threadIdx.x;
  const int per = (t + kSlotThreads - 1) / kSlotThreads;
  const int t0 = tid * per, t1 = min(t, t0 + per);
  const long long n = (long long)b * t, total = (long long)n_exp * b * cap;
  for (int e = 0; e < n_exp; ++e) cnt[e][tid] = 0;
  // empty slots of this sequence
  for (int i = tid; i < n_exp * cap; i += kSlotThreads) {
    const int e = i / cap, c = i - e * cap;
    tok[((long long)e * b + row) * cap + c] = n;
  }
  for (int tt = t0; tt < t1; ++tt)
    for (int j = 0; j < k; ++j) cnt[(int)idx[((long long)row * t + tt) * k + j]][tid] += 1;
  __syncthreads();
  // exclusive scan over the 256 chunk counts of each expert: one warp per expert at a time
  const int warp = tid >> 5, lane = tid & 31;
  for (int e = warp; e < n_exp; e += kSlotThreads / 32) {
    int v[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = cnt[e][lane * 8 + i]; sum += v[i]; }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    int run = incl - sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) { cnt[e][lane * 8 + i] = (unsigned short)min(run, 65535); run += v[i]; }
  }
  __syncthreads();
  for (int tt = t0; tt < t1; ++tt) {
    const long long token = (long long)row * t + tt;
    for (int j = 0; j < k; ++j) {
      const int e = (int)idx[token * k + j];
      const int pos = cnt[e][tid];
      cnt[e][tid] = (unsigned short)min(pos + 1, 65535);
      long long s = total;
      if (pos < cap) {
        s = ((long long)e * b + row) * cap + pos;
        tok[s] = token;
      }
      slot[token * k + j] = s;
    }
  }
}

// Backward of the gate-weighted combine: dys[slot[n,k]] = gates[n,k] * dout[n] (slots are unique; empty slots stay at
// the zero the caller wrote) and dgates[n,k] = <ys[slot[n,k]], dout[n]>.  One warp per token.
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ ys, const long long* __restrict__ slot, const float* __restrict__ gates,
                                       const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dys, float* __restrict__ dgates,
                                       int n, int C, int topk, long long S) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  for (int kk = 0; kk < topk; ++kk) {
    const long long s = slot[(size_t)row * topk + kk];
    float acc = 0.f;
    if (s >= 0 && s < S) {
      const float g = gates[(size_t)row * topk + kk];
      for (int c = lane * 8; c < C; c += 256) {
        const uint4 uy = *reinterpret_cast<const uint4*>(ys + (size_t)s * C + c);
        const uint4 ud = *reinterpret_cast<const uint4*>(dout + (size_t)row * C + c);
        const uint32_t wy[4] = {uy.x, uy.y, uy.z, uy.w}, wd[4] = {ud.x, ud.y, ud.z, ud.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fy = unpack_bf16(wy[i]), fd = unpack_bf16(wd[i]);
          acc += fy.x * fd.x + fy.y * fd.y;
          o[i] = pack_bf16(g * fd.x, g * fd.y);
        }
        *reinterpret_cast<uint4*>(dys + (size_t)s * C + c) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dgates[(size_t)row * topk + kk] = acc;
  }
}

// Up to two auxiliary targets per row (multi-token prediction: the tokens two and three positions ahead) share the
// row's soft-max: nll_aux = sum_k w_k * (lse - z[target_k]) and the logit gradient gains w_k * (p - onehot_k).
struct AuxTargets {
  const long long* tg[2];
  const float* w[2];        // absolute row weights (0 where the auxiliary target does not apply)
  float* nll_aux;           // [M], written when any auxiliary target is given
  float smooth;             // label smoothing of the main target: loss = (1 - s) * nll + s * (lse - mean_v z_v)
};

// Softcap cross-entropy over full rows of bf16 logits [M, ldl] (first V columns valid), one CTA per row.
//   z = cap * tanh(l / cap);  lse = log sum exp z;  nll = lse - z[target]
// Outputs: nll[row] (0 where target < 0).  With `dlogits` (may alias logits) the gradient of
//   sum_rows w_row * nll_row,   w_row = row_w ? row_w[row] : 1/max(1, *n_valid) / loss_div
// is written in place: d l = w * (softmax(z) - onehot) * (1 - tanh^2).  Bounded logits (|z| <= cap) make a max pass
// unnecessary: exp(z - cap) never overflows.
__global__ void softcap_ce_kernel(const __nv_bfloat16* logits, long long ldl, const long long* targets, int V, float cap, float* nll,
                                  __nv_bfloat16* dlogits, const float* row_w, const float* n_valid, float inv_loss_div, int M, int capped,
                                  AuxTargets aux) {
  const int row = blockIdx.x;
  if (row >= M) return;
  const __nv_bfloat16* l = logits + (size_t)row * ldl;
  const long long tgt = targets[row];
  const float inv_cap = 1.0f / cap;
  __shared__ float red[32], red_t[32];
  __shared__ float s_total, s_tsum;
  float s = 0.f, st = 0.f;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(l + c);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 f = unpack_bf16(w[t]);
      const float t0 = capped ? f.x * inv_cap : tanhf(f.x * inv_cap), t1 = capped ? f.y * inv_cap : tanhf(f.y * inv_cap);
      s += __expf(cap * t0 - cap) + __expf(cap * t1 - cap);
      st += t0 + t1;
    }
  }
  s = warp_sum(s);
  st = warp_sum(st);
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = s; red_t[threadIdx.x >> 5] = st; }
  const bool valid = tgt >= 0 && tgt < V;
  long long t2 = -1, t3 = -1;
  float a2 = 0.f, a3 = 0.f;
  if (aux.tg[0]) { t2 = aux.tg[0][row]; a2 = (t2 >= 0 && t2 < V) ? aux.w[0][row] : 0.f; }
  if (aux.tg[1]) { t3 = aux.tg[1][row]; a3 = (t3 >= 0 && t3 < V) ? aux.w[1][row] : 0.f; }
  // the target logits are read here, before the barriers: the gradient may be written over the logits (in place), and
  // no thread stores before the second barrier
  float z_tgt = 0.f, z_2 = 0.f, z_3 = 0.f;
  if (threadIdx.x == 0) {
    if (valid) z_tgt = __bfloat162float(l[tgt]);
    if (a2 != 0.f) z_2 = __bfloat162float(l[t2]);
    if (a3 != 0.f) z_3 = __bfloat162float(l[t3]);
    if (!capped) { z_tgt = cap * tanhf(z_tgt * inv_cap); z_2 = cap * tanhf(z_2 * inv_cap); z_3 = cap * tanhf(z_3 * inv_cap); }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    float vt = threadIdx.x < (blockDim.x >> 5) ? red_t[threadIdx.x] : 0.f;
    v = warp_sum(v);
    vt = warp_sum(vt);
    if (threadIdx.x == 0) { s_total = v; s_tsum = vt; }
  }
  __syncthreads();
  const float lse = logf(s_total) + cap;
  const float sm = aux.smooth, mean_z = cap * s_tsum / (float)V;
  if (threadIdx.x == 0) {
    float out = 0.f;
    if (valid) out = lse - (1.0f - sm) * z_tgt - sm * mean_z;
    nll[row] = out;
  }
  if (threadIdx.x == 0 && aux.nll_aux) {
    float out = 0.f;
    if (a2 != 0.f) out += a2 * (lse - z_2);
    if (a3 != 0.f) out += a3 * (lse - z_3);
    aux.nll_aux[row] = out;
  }
  if (!dlogits) return;
  float w = 0.f;
  if (valid) w = row_w ? row_w[row] : inv_loss_div / fmaxf(1.0f, *n_valid);
  const float wsum = w + a2 + a3;
  const float w_tgt = w * (1.0f - sm), w_uni = w * sm / (float)V;
  __nv_bfloat16* d = dlogits + (size_t)row * ldl;
  for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(l + c);
    const uint32_t wd[4] = {u.x, u.y, u.z, u.w};
    float g[8];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 f = unpack_bf16(wd[t]);
      const float t0 = capped ? f.x * inv_cap : tanhf(f.x * inv_cap), t1 = capped ? f.y * inv_cap : tanhf(f.y * inv_cap);
      float p0 = wsum * __expf(cap * t0 - lse) - w_uni, p1 = wsum * __expf(cap * t1 - lse) - w_uni;
      const int c0i = c + 2 * t, c1i = c0i + 1;
      if (c0i == tgt) p0 -= w_tgt;
      if (c1i == tgt) p1 -= w_tgt;
      if (c0i == t2) p0 -= a2;
      if (c1i == t2) p1 -= a2;
      if (c0i == t3) p0 -= a3;
      if (c1i == t3) p1 -= a3;
      g[2 * t] = p0 * (1.0f - t0 * t0);
      g[2 * t + 1] = p1 * (1.0f - t1 * t1);
    }
    uint4 o;
    o.x = pack_bf16(g[0], g[1]); o.y = pack_bf16(g[2], g[3]); o.z = pack_bf16(g[4], g[5]); o.w = pack_bf16(g[6], g[7]);
    *reinterpret_cast<uint4*>(d + c) = o;
  }
  // padded vocabulary columns carry no gradient
  for (int c = V + threadIdx.x; c < ldl; c += blockDim.x) d[c] = __float2bfloat16(0.f);
}

// Same contract for V <= 65536 with one 1024-thread block per row: the row is read once, tanh(l / cap) of the thread's 64
// columns stays in registers as fp16 pairs between the two passes, and the transcendental work is three special-function
// operations per element (tanh.approx, ex2 for the sum, ex2 for the probability) instead of two libm tanhf and two expf.
// tanh.approx and fp16 storage both carry about 2^-11 relative error, below the bf16 rounding of the logits themselves.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Second pass of the row kernel for one thread: gradient of its 64 columns from the saved tanh values.
// p = exp2(k2 * t - lw) already carries the row's weight (lw = lse2 - log2(weight sum)).  FIX: this thread owns the column
// of a target (at most three threads of a row do) and subtracts the target weights; the others never compare.
template <bool FIX>
__device__ __forceinline__ void ce_row_grad(const __half2 (&th)[8][4], __nv_bfloat16* d, int V, float k2, float lw, float w_uni, int tg, float w_tgt,
                                            int t2, float a2, int t3, float a3) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = (i * 1024 + threadIdx.x) * 8;
    if (c >= V) continue;
    float g[8];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 tt = __half22float2(th[i][t]);
      float p0 = ex2_fast(fmaf(k2, tt.x, -lw)) - w_uni, p1 = ex2_fast(fmaf(k2, tt.y, -lw)) - w_uni;
      if (FIX) {
        const int c0i = c + 2 * t, c1i = c0i + 1;
        if (c0i == tg) p0 -= w_tgt;
        if (c1i == tg) p1 -= w_tgt;
        if (c0i == t2) p0 -= a2;
        if (c1i == t2) p1 -= a2;
        if (c0i == t3) p0 -= a3;
        if (c1i == t3) p1 -= a3;
      }
      g[2 * t] = p0 * fmaf(-tt.x, tt.x, 1.0f);
      g[2 * t + 1] = p1 * fmaf(-tt.y, tt.y, 1.0f);
    }
    uint4 o;
    o.x = pack_bf16(g[0], g[1]); o.y = pack_bf16(g[2], g[3]); o.z = pack_bf16(g[4], g[5]); o.w = pack_bf16(g[6], g[7]);
    *reinterpret_cast<uint4*>(d + c) = o;
  }
}

// Row kernel for vocabularies of 8192 .. 65536: persistent, one CTA of 1024 threads per SM walking rows.  A row's logits
// arrive as four bulk asynchronous copies (quarter rows of up to 32 KB) in shared memory, each signalled by an mbarrier.
// A thread takes its 16 values of a quarter into registers (as tanh values in half precision); the last of the CTA's 32
// warps to have done so hands the quarter straight back to the copy engine for the CTA's next row, so reads are in
// flight through both passes of a row (sum of exponentials; probabilities, gradient and stores).  With a CTA per row and
// plain loads the row's read, its two exponential passes (2 x 65536 results at 16 per clock) and its write ran one
// after the other, about 17 000 clocks per row where each alone needs 8 000 to 9 000.
constexpr int CE_Q_COLS = 16384;
constexpr int CE_SMEM_BYTES = 4 * CE_Q_COLS * 2 + 64;
// Second pass for logits that the GEMM epilogue already soft-capped (z = cap * tanh(. / cap) as stored): the thread kept
// its 64 logits as the bf16 pairs they arrived as, so there is no conversion on either side; p = exp2(z log2(e) - lw),
// d tanh = 1 - (z / cap)^2.  SMOOTH: label smoothing's uniform term is live.
template <bool FIX, bool SMOOTH>
__device__ __forceinline__ void ce_row_grad_capped(const uint32_t (&zw)[8][4], __nv_bfloat16* d, int V, float nic2, float lw, float w_uni,
                                                   int tg, float w_tgt, int t2, float a2, int t3, float a3) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = (i * 1024 + threadIdx.x) * 8;
    if (c >= V) continue;
    uint32_t o[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float z0 = __uint_as_float(zw[i][t] << 16), z1 = __uint_as_float(zw[i][t] & 0xffff0000u);
      float p0 = ex2_fast(fmaf(z0, 1.4426950408889634f, -lw)), p1 = ex2_fast(fmaf(z1, 1.4426950408889634f, -lw));
      if (SMOOTH) { p0 -= w_uni; p1 -= w_uni; }
      if (FIX) {
        const int c0i = c + 2 * t, c1i = c0i + 1;
        if (c0i == tg) p0 -= w_tgt;
        if (c1i == tg) p1 -= w_tgt;
        if (c0i == t2) p0 -= a2;
        if (c1i == t2) p1 -= a2;
        if (c0i == t3) p0 -= a3;
        if (c1i == t3) p1 -= a3;
      }
      o[t] = pack_bf16(p0 * fmaf(z0 * nic2, z0, 1.0f), p1 * fmaf(z1 * nic2, z1, 1.0f));
    }
    *reinterpret_cast<uint4*>(d + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <bool CAPPED>
__global__ void __launch_bounds__(1024, 1)
softcap_ce_row_kernel(const __nv_bfloat16* __restrict__ logits, long long ldl, const long long* __restrict__ targets, int V, float cap,
                      float* __restrict__ nll, __nv_bfloat16* dlogits, const float* __restrict__ row_w, const float* __restrict__ n_valid,
                      float inv_loss_div, int M, AuxTargets aux, int* err) {
  constexpr bool capped = CAPPED;
  extern __shared__ __align__(128) uint8_t ce_smem[];
  __shared__ float red[32], red_t[32];
  __shared__ float s_total, s_tsum;
  __shared__ int s_abort, s_taken[4];
  const uint32_t buf = smem_u32(ce_smem), bar = buf + 4u * CE_Q_COLS * 2u;
  const float inv_cap = 1.0f / cap, k2 = cap * 1.4426950408889634f;
  if (threadIdx.x == 0) {
    s_abort = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) { mbar_init(bar + 8u * q, 1); s_taken[q] = 0; }
    fence_barrier_init();
  }
  __syncthreads();
  auto issue = [&](int row, int q) {                            // one thread: quarter q of a row
    const int cols = min(V - q * CE_Q_COLS, CE_Q_COLS);
    if (cols <= 0) return;
    mbar_arrive_expect_tx(bar + 8u * q, (uint32_t)cols * 2u);
    bulk_load(buf + (uint32_t)(q * CE_Q_COLS * 2), logits + (size_t)row * ldl + q * CE_Q_COLS, (uint32_t)cols * 2u, bar + 8u * q);
  };
  if (threadIdx.x == 0 && (int)blockIdx.x < M) {
#pragma unroll
    for (int q = 0; q < 4; ++q) issue(blockIdx.x, q);
  }
  const __nv_bfloat16* sl = reinterpret_cast<const __nv_bfloat16*>(ce_smem);
  int n = 0;
  for (int row = blockIdx.x; row < M; row += gridDim.x, ++n) {
    const long long tgt = targets[row];
    const bool valid = tgt >= 0 && tgt < V;
    long long t2 = -1, t3 = -1;
    float a2 = 0.f, a3 = 0.f;
    if (aux.tg[0]) { t2 = aux.tg[0][row]; a2 = (t2 >= 0 && t2 < V) ? aux.w[0][row] : 0.f; }
    if (aux.tg[1]) { t3 = aux.tg[1][row]; a3 = (t3 >= 0 && t3 < V) ? aux.w[1][row] : 0.f; }
    // what a thread keeps of its 64 logits between the passes: the bf16 pairs themselves (already capped), or the tanh
    // values as half pairs
    uint32_t keep[8][4];
    float s = 0.f, st = 0.f;                                    // sum of exponentials; sum of tanh values (of logits when capped)
    float z_tgt = 0.f, z_2 = 0.f, z_3 = 0.f;
    bool ok = true;
    const bool smoothing = aux.smooth != 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const bool live = V > q * CE_Q_COLS;                      // uniform
      if (live) ok = ok && mbar_wait(bar + 8u * q, (uint32_t)(n & 1), &s_abort, err, ERR_WAIT_FULL);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int i = q * 2 + j;
        const int c = (i * 1024 + threadIdx.x) * 8;
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (c < V && ok) raw = *reinterpret_cast<const uint4*>(ce_smem + (size_t)c * 2);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        if (capped) {
          // the GEMM epilogue already applied cap * tanh(. / cap): exp2(k2 t - k2) = exp2(z log2(e) - k2)
#pragma unroll
          for (int t = 0; t < 4; ++t) keep[i][t] = w[t];
          if (c < V) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float z0 = __uint_as_float(w[t] << 16), z1 = __uint_as_float(w[t] & 0xffff0000u);
              s += ex2_fast(fmaf(z0, 1.4426950408889634f, -k2)) + ex2_fast(fmaf(z1, 1.4426950408889634f, -k2));
              if (smoothing) st += z0 + z1;
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float t0 = tanh_fast(__uint_as_float(w[t] << 16) * inv_cap), t1 = tanh_fast(__uint_as_float(w[t] & 0xffff0000u) * inv_cap);
            const __half2 hh = __floats2half2_rn(t0, t1);
            keep[i][t] = *reinterpret_cast<const uint32_t*>(&hh);
            if (c < V) {
              s += ex2_fast(fmaf(k2, t0, -k2)) + ex2_fast(fmaf(k2, t1, -k2));
              st += t0 + t1;
            }
          }
        }
      }
      if (live) {
        // the target logits come from the row buffer while it still holds this row: the gradient may overwrite the
        // logits in global memory, and the quarter is refilled once every warp has taken it
        if (threadIdx.x == 0 && ok) {
          if (valid && (int)(tgt / CE_Q_COLS) == q) z_tgt = __bfloat162float(sl[tgt]);
          if (a2 != 0.f && (int)(t2 / CE_Q_COLS) == q) z_2 = __bfloat162float(sl[t2]);
          if (a3 != 0.f && (int)(t3 / CE_Q_COLS) == q) z_3 = __bfloat162float(sl[t3]);
        }
        __threadfence_block();                                  // this thread's reads of the quarter are done
        __syncwarp();
        if ((threadIdx.x & 31) == 0 && atomicAdd(&s_taken[q], 1) == 31) {
          s_taken[q] = 0;                                       // last of the 32 warps: the quarter is free
          if (ok && row + (int)gridDim.x < M) {
            fence_proxy_async_smem();
            issue(row + gridDim.x, q);
          }
        }
      }
    }
    if (!capped) { z_tgt = cap * tanh_fast(z_tgt * inv_cap); z_2 = cap * tanh_fast(z_2 * inv_cap); z_3 = cap * tanh_fast(z_3 * inv_cap); }
    s = warp_sum(s);
    st = warp_sum(st);
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = s; red_t[threadIdx.x >> 5] = st; }
    if (!__syncthreads_and(ok ? 1 : 0)) break;
    if (threadIdx.x < 32) {
      float v = red[threadIdx.x], vt = red_t[threadIdx.x];
      v = warp_sum(v);
      vt = warp_sum(vt);
      if (threadIdx.x == 0) { s_total = v; s_tsum = vt; }
    }
    __syncthreads();
    const float lse2 = log2f(s_total) + k2;          // log-sum-exp in base-2 units
    const float sm = aux.smooth, mean_z = (capped ? 1.0f : cap) * s_tsum / (float)V;
    if (threadIdx.x == 0) {
      float out = 0.f;
      if (valid) out = lse2 * 0.6931471805599453f - (1.0f - sm) * z_tgt - sm * mean_z;
      nll[row] = out;
      if (aux.nll_aux) {
        const float lse = lse2 * 0.6931471805599453f;
        float oa = 0.f;
        if (a2 != 0.f) oa += a2 * (lse - z_2);
        if (a3 != 0.f) oa += a3 * (lse - z_3);
        aux.nll_aux[row] = oa;
      }
    }
    if (!dlogits) continue;
    float w = 0.f;
    if (valid) w = row_w ? row_w[row] : inv_loss_div / fmaxf(1.0f, *n_valid);
    const float wsum = w + a2 + a3;
    const float w_tgt = w * (1.0f - sm), w_uni = w * sm / (float)V;
    // a row without any live target has weight sum 0: lw = +inf makes every probability term exactly 0
    const float lw = wsum > 0.f ? lse2 - log2f(wsum) : __int_as_float(0x7f800000);
    const int tgi = (valid && w_tgt != 0.f) ? (int)tgt : -1, t2i = a2 != 0.f ? (int)t2 : -1, t3i = a3 != 0.f ? (int)t3 : -1;
    // thread x holds columns (i * 1024 + x) * 8 .. + 7, so column c belongs to thread (c >> 3) & 1023
    const int me = threadIdx.x;
    const bool owner = (tgi >= 0 && ((tgi >> 3) & 1023) == me) || (t2i >= 0 && ((t2i >> 3) & 1023) == me) ||
                       (t3i >= 0 && ((t3i >> 3) & 1023) == me);
    __nv_bfloat16* d = dlogits + (size_t)row * ldl;
    if (capped) {
      const float nic2 = -inv_cap * inv_cap;
      if (owner) ce_row_grad_capped<true, true>(keep, d, V, nic2, lw, w_uni, tgi, w_tgt, t2i, a2, t3i, a3);
      else if (smoothing) ce_row_grad_capped<false, true>(keep, d, V, nic2, lw, w_uni, tgi, w_tgt, t2i, a2, t3i, a3);
      else ce_row_grad_capped<false, false>(keep, d, V, nic2, lw, w_uni, tgi, w_tgt, t2i, a2, t3i, a3);
    } else {
      const __half2 (&th)[8][4] = reinterpret_cast<const __half2 (&)[8][4]>(keep);
      if (owner) ce_row_grad<true>(th, d, V, k2, lw, w_uni, tgi, w_tgt, t2i, a2, t3i, a3);
      else ce_row_grad<false>(th, d, V, k2, lw, w_uni, tgi, w_tgt, t2i, a2, t3i, a3);
    }
    for (int c = V + threadIdx.x; c < ldl; c += blockDim.x) d[c] = __float2bfloat16(0.f);
  }
  // a CTA that gave up may still have a copy on its way into shared memory: stay a moment before the memory goes
  if (s_abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

// y = cap * tanh(x / cap) in fp32 from bf16 logits, first V of ldl columns
__global__ void softcap_logits_kernel(const __nv_bfloat16* logits, long long ldl, float* out, int V, float cap, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long r = i / V;
  const int c = (int)(i - r * V);
  out[i] = cap * tanhf(__bfloat162float(logits[r * ldl + c]) / cap);
}

// fused AdamW on fp32 master + moments with a low-precision replica write (decoupled decay, bias correction)
__global__ void adamw_kernel(float* p, const float* g, float* m, float* v, __nv_bfloat16* replica, long long n, float lr, float b1,
                             float b2, float eps, float wd, float c1, float c2, float gscale, const float* ok) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gi = g[i] * gscale;
  if (ok && *ok <= 0.f) gi = 0.f;
  float pi = p[i] * (1.0f - lr * wd);
  const float mi = m[i] + (1.0f - b1) * (gi - m[i]);
  const float vi = v[i] + (1.0f - b2) * (gi * gi - v[i]);
  pi -= lr * (mi / c1) / (sqrtf(vi / c2) + eps);
  p[i] = pi; m[i] = mi; v[i] = vi;
  if (replica) replica[i] = __float2bfloat16(pi);
}

// sparse Adam on touched table rows: table[rows[i]] (bf16) updated from g[i], m[i], v[i] (fp32, compacted)
__global__ void sparse_adam_kernel(__nv_bfloat16* table, const long long* rows, const float* g, float* m, float* v, int n, int C, float lr,
                                   float b1, float b2, float eps, float decay, float c1, float c2) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  __nv_bfloat16* w = table + (size_t)rows[row] * C;
  for (int c = lane; c < C; c += 32) {
    const size_t i = (size_t)row * C + c;
    const float gi = g[i];
    const float mi = m[i] + (1.0f - b1) * (gi - m[i]);
    const float vi = v[i] + (1.0f - b2) * (gi * gi - v[i]);
    m[i] = mi; v[i] = vi;
    const float wi = __bfloat162float(w[c]) * (1.0f - lr * decay) - lr * (mi / c1) / (sqrtf(vi / c2) + eps);
    w[c] = __float2bfloat16(wi);
  }
}

}  // namespace bones

extern "C" {
using namespace bones;
#define ROWS_PER_BLOCK 8
#define ROW_GRID(M) dim3(((M) + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK), dim3(ROWS_PER_BLOCK * 32)

int bones_rmsnorm_fwd(const void* x, void* y, int M, int C, void* stream) {
  if (C % 8 || C > kMaxVec * 256) return -2;
  rmsnorm_fwd_kernel<<<ROW_GRID(M), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, M, C);
  return (int)cudaGetLastError();
}
int bones_rmsnorm_bwd(const void* x, const void* dy, const void* add, void* dx, int M, int C, void* stream) {
  if (C % 8 || C > kMaxVec * 256) return -2;
#define BONES_RMS_BWD_CASE(NV)                                                                                                  \
  case NV:                                                                                                                      \
    rmsnorm_bwd_packed_kernel<NV><<<ROW_GRID(M), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,  \
                                                                            (const __nv_bfloat16*)add, (__nv_bfloat16*)dx, M);  \
    return (int)cudaGetLastError();
  if (C % 256 == 0) {
    switch (C / 256) {
      BONES_RMS_BWD_CASE(2) BONES_RMS_BWD_CASE(3) BONES_RMS_BWD_CASE(4) BONES_RMS_BWD_CASE(5) BONES_RMS_BWD_CASE(6)
      default: break;
    }
  }
  rmsnorm_bwd_kernel<<<ROW_GRID(M), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)add,
                                                             (__nv_bfloat16*)dx, M, C);
  return (int)cudaGetLastError();
}
int bones_resid_mix_norm_fwd(const void* x, const void* x0, const float* a, const float* b, void* xm, void* xn, int M, int C, void* stream) {
  if (C % 8 || C > kMaxVec * 256) return -2;
  resid_mix_norm_fwd_kernel<<<ROW_GRID(M), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, a, b,
                                                                    (__nv_bfloat16*)xm, (__nv_bfloat16*)xn, M, C);
  return (int)cudaGetLastError();
}
int bones_resid_mix_norm_bwd(const void* x, const void* x0, const void* xm, const float* a, const float* b, const void* dxm, const void* dxn,
                             void* dx, void* dx0, float* da, float* db, int M, int C, int acc_x0, void* stream) {
  if (C % 8 || C > kMaxVec * 256) return -2;
#define BONES_MIX_BWD_CASE(NV)                                                                                                   \
  case NV:                                                                                                                       \
    resid_mix_norm_bwd_packed_kernel<NV><<<ROW_GRID(M), 0, (cudaStream_t)stream>>>(                                              \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, (const __nv_bfloat16*)xm, a, b, (const __nv_bfloat16*)dxm,            \
        (const __nv_bfloat16*)dxn, (__nv_bfloat16*)dx, (__nv_bfloat16*)dx0, da, db, M, acc_x0);                                  \
    return (int)cudaGetLastError();
  if (C % 256 == 0) {
    switch (C / 256) {
      BONES_MIX_BWD_CASE(2) BONES_MIX_BWD_CASE(3) BONES_MIX_BWD_CASE(4) BONES_MIX_BWD_CASE(5) BONES_MIX_BWD_CASE(6)
      default: break;
    }
  }
  resid_mix_norm_bwd_kernel<<<ROW_GRID(M), 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)x0, (const __nv_bfloat16*)xm, a, b, (const __nv_bfloat16*)dxm, (const __nv_bfloat16*)dxn,
      (__nv_bfloat16*)dx, (__nv_bfloat16*)dx0, da, db, M, C, acc_x0);
  return (int)cudaGetLastError();
}
int bones_gather_rows(const void* table, const void* idx, int idx_is_64, void* out, int n, int C, long long n_rows, void* stream) {
  if (C % 8) return -2;
  if (idx_is_64)
    gather_rows_kernel<long long><<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)table, (const long long*)idx,
                                                                          (__nv_bfloat16*)out, n, C, n_rows);
  else
    gather_rows_kernel<int><<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)table, (const int*)idx, (__nv_bfloat16*)out, n, C,
                                                                    n_rows);
  return (int)cudaGetLastError();
}
int bones_scatter_add_rows(const void* dy, const void* idx, int idx_is_64, float* grad, int n, int C, long long n_rows, void* stream) {
  if (C % 8) return -2;
  if (idx_is_64)
    scatter_add_rows_kernel<long long><<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const long long*)idx, grad, n, C,
                                                                               n_rows);
  else
    scatter_add_rows_kernel<int><<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const int*)idx, grad, n, C, n_rows);
  return (int)cudaGetLastError();
}
int bones_moe_combine(const void* ys, const long long* slot, const float* gates, void* out, int n, int C, int topk, long long S, void* stream) {
  if (C % 8) return -2;
  moe_combine_kernel<<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)ys, slot, gates, (__nv_bfloat16*)out, n, C, topk, S);
  return (int)cudaGetLastError();
}
int bones_moe_slots(const long long* idx, long long* slot, long long* tok, int b, int t, int k, int n_exp, int cap, void* stream) {
  if (n_exp > kMaxExperts || t > 8 * kSlotThreads * 32) return -2;
  moe_slots_kernel<<<b, kSlotThreads, 0, (cudaStream_t)stream>>>(idx, slot, tok, b, t, k, n_exp, cap);
  return (int)cudaGetLastError();
}
int bones_moe_combine_bwd(const void* ys, const long long* slot, const float* gates, const void* dout, void* dys, float* dgates, int n, int C,
                          int topk, long long S, void* stream) {
  if (C % 8) return -2;
  moe_combine_bwd_kernel<<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)ys, slot, gates, (const __nv_bfloat16*)dout,
                                                                 (__nv_bfloat16*)dys, dgates, n, C, topk, S);
  return (int)cudaGetLastError();
}
int bones_softcap_ce(const void* logits, long long ldl, const long long* targets, int V, float cap, float* nll, void* dlogits,
                     const float* row_w, const float* n_valid, float inv_loss_div, int M, int capped, const long long* tg2, const float* w2,
                     const long long* tg3, const float* w3, float* nll_aux, float label_smoothing, void* stream) {
  if (V % 8 || ldl % 8) return -2;
  AuxTargets aux;
  aux.tg[0] = tg2; aux.w[0] = w2; aux.tg[1] = tg3; aux.w[1] = w3; aux.nll_aux = nll_aux;
  aux.smooth = label_smoothing;
  if (V <= 65536 && V >= 8192 && ((uintptr_t)logits % 16) == 0) {
    static bool attr_set = false;
    if (!attr_set) {
      BONES_CHECK(cudaFuncSetAttribute(softcap_ce_row_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, CE_SMEM_BYTES));
      BONES_CHECK(cudaFuncSetAttribute(softcap_ce_row_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, CE_SMEM_BYTES));
      attr_set = true;
    }
    int dev = 0, sms = 0;
    BONES_CHECK(cudaGetDevice(&dev));
    BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int grid = M < sms ? M : sms;
    if (grid <= 0) return 0;
    if (capped)
      softcap_ce_row_kernel<true><<<grid, 1024, CE_SMEM_BYTES, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)logits, ldl, targets, V, cap, nll, (__nv_bfloat16*)dlogits, row_w, n_valid, inv_loss_div, M, aux, error_word());
    else
      softcap_ce_row_kernel<false><<<grid, 1024, CE_SMEM_BYTES, (cudaStream_t)stream>>>(
          (const __nv_bfloat16*)logits, ldl, targets, V, cap, nll, (__nv_bfloat16*)dlogits, row_w, n_valid, inv_loss_div, M, aux, error_word());
    return (int)cudaGetLastError();
  }
  softcap_ce_kernel<<<M, 512, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ldl, targets, V, cap, nll, (__nv_bfloat16*)dlogits,
                                                        row_w, n_valid, inv_loss_div, M, capped, aux);
  return (int)cudaGetLastError();
}
int bones_softcap_logits(const void* logits, long long ldl, float* out, int V, float cap, long long rows, void* stream) {
  const long long total = rows * V;
  softcap_logits_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ldl, out, V, cap, total);
  return (int)cudaGetLastError();
}
int bones_adamw(float* p, const float* g, float* m, float* v, void* replica, long long n, float lr, float b1, float b2, float eps, float wd,
                int step, float gscale, const float* ok, void* stream) {
  const float c1 = 1.0f - powf(b1, (float)step), c2 = 1.0f - powf(b2, (float)step);
  adamw_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p, g, m, v, (__nv_bfloat16*)replica, n, lr, b1, b2, eps, wd, c1, c2,
                                                                            gscale, ok);
  return (int)cudaGetLastError();
}
int bones_sparse_adam(void* table, const long long* rows, const float* g, float* m, float* v, int n, int C, float lr, float b1, float b2,
                      float eps, float decay, int step, void* stream) {
  const float c1 = 1.0f - powf(b1, (float)step), c2 = 1.0f - powf(b2, (float)step);
  sparse_adam_kernel<<<ROW_GRID(n), 0, (cudaStream_t)stream>>>((__nv_bfloat16*)table, rows, g, m, v, n, C, lr, b1, b2, eps, decay, c1, c2);
  return (int)cudaGetLastError();
}
}  // extern "C"
BONES_BOUNDS_EXPORT(elementwise)
