// Causal flash attention for the decoder, forward pass, on tcgen05 tensor cores with TMEM accumulators and TMA loads,
// plus the RoPE + QK-RMSNorm pre/post passes.
//
// Semantics (reference: fused RoPE + QK-norm + causal attention, round2/source/kernels/nki_attn_bandpro.py:686-978; eager
// form round2/source/train.py:10209-10252): q and k are rotated (rotate-half RoPE), RMS-normalised per head, and
// attention is causal softmax(scale * q k^T) v.  Added here: keys are limited to the query's document
// (`doc_start[b, t]` = position of the most recent BOS) and, for banded layers, to the query's 128-token tile and the
// `window_tiles - 1` tiles before it (the reference's tile band, round2/source/train.py:4740-4745).
//
// Because q and k are RMS-normalised, |q.k| <= head_dim, so the softmax uses the fixed shift `scale * head_dim` instead
// of a running maximum (the reference kernels do the same): P = exp(scale*s - scale*D) never overflows and no rescale of
// the output accumulator is ever needed.  The row sum is kept in registers and `lse = log(sum) + scale*D` is saved.
//
// One CTA per (128-query tile, head, batch).  Warp 0: TMA producer (Q once, K/V tiles through a 2-stage ring).  Warp 1:
// tcgen05.mma issuer: S = Q K^T into one of two TMEM buffers, then O += P V with P read from shared memory.  Warps 2-5:
// one query row per thread: tcgen05.ld the scores, mask, exponentiate, write P (bf16) into 128-byte-swizzled shared
// memory for the second MMA; at the end divide O by the row sum and store.
#include "common.cuh"

namespace bones {

constexpr float kQkEps = 1.1920928955078125e-07f;   // 2^-23

// ---------------------------------------------------------------------------------------------------------------
// RoPE + QK-norm pre-pass: qkv [M, 3A] -> qk [M, 2A]  (A = H * D; q-hat then k-hat).  One warp per (row, head, q|k).
// ---------------------------------------------------------------------------------------------------------------
template <int D>
__global__ void rope_qknorm_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                                       const float* __restrict__ sinT, __nv_bfloat16* __restrict__ qk, long long M, int T, int H) {
  constexpr int HALF = D / 2, PER = HALF / 32;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= M * H * 2) return;
  const int which = (int)(w % 2), h = (int)((w / 2) % H);
  const long long row = w / (2 * H);
  const int t = (int)(row % T);
  const long long A = (long long)H * D;
  const __nv_bfloat16* src = qkv + row * 3 * A + which * A + (long long)h * D;
  __nv_bfloat16* dst = qk + row * 2 * A + which * A + (long long)h * D;
  float y1[PER], y2[PER], ss = 0.f;
  float x1[PER], x2[PER], cs[PER], sn[PER];
  if constexpr (PER == 2) {   // 4-byte / 8-byte vector accesses: a warp reads 128 contiguous bytes per half
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 2 * lane));
    const float2 c2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + HALF + 2 * lane));
    const float2 cc = *reinterpret_cast<const float2*>(cosT + (long long)t * HALF + 2 * lane);
    const float2 sc = *reinterpret_cast<const float2*>(sinT + (long long)t * HALF + 2 * lane);
    x1[0] = a.x; x1[1] = a.y; x2[0] = c2.x; x2[1] = c2.y; cs[0] = cc.x; cs[1] = cc.y; sn[0] = sc.x; sn[1] = sc.y;
  } else {
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = lane * PER + e;
      x1[e] = __bfloat162float(src[i]); x2[e] = __bfloat162float(src[HALF + i]);
      cs[e] = cosT[(long long)t * HALF + i]; sn[e] = sinT[(long long)t * HALF + i];
    }
  }
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    y1[e] = x1[e] * cs[e] + x2[e] * sn[e];
    y2[e] = -x1[e] * sn[e] + x2[e] * cs[e];
    ss += y1[e] * y1[e] + y2[e] * y2[e];
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + kQkEps);
  if constexpr (PER == 2) {
    *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(y1[0] * r, y1[1] * r);
    *reinterpret_cast<__nv_bfloat162*>(dst + HALF + 2 * lane) = __floats2bfloat162_rn(y2[0] * r, y2[1] * r);
  } else {
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = lane * PER + e;
      dst[i] = __float2bfloat16(y1[e] * r);
      dst[HALF + i] = __float2bfloat16(y2[e] * r);
    }
  }
}

// Backward of the pre-pass: dq-hat/dk-hat (fp32 [M, 2A]) + dv (bf16 [M, A]) -> dqkv (bf16 [M, 3A]).
// u = rope(x), r = rsqrt(mean(u^2)+eps), xhat = u r;  du = r (dxhat - xhat mean(dxhat xhat));  dx = rope^T(du).
template <int D>
__global__ void rope_qknorm_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                                       const float* __restrict__ sinT, const float* __restrict__ dqk,
                                       const __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ dqkv, long long M, int T,
                                       int H) {
  constexpr int HALF = D / 2, PER = HALF / 32;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= M * H * 3) return;
  const int which = (int)(w % 3), h = (int)((w / 3) % H);
  const long long row = w / (3 * H);
  const long long A = (long long)H * D;
  __nv_bfloat16* out = dqkv + row * 3 * A + which * A + (long long)h * D;
  if (which == 2) {   // values pass straight through
    const __nv_bfloat16* g = dv + row * A + (long long)h * D;
    if constexpr (D == 128) {
      *reinterpret_cast<uint2*>(out + 4 * lane) = *reinterpret_cast<const uint2*>(g + 4 * lane);
    } else {
      for (int i = lane; i < D; i += 32) out[i] = g[i];
    }
    return;
  }
  const int t = (int)(row % T);
  const __nv_bfloat16* src = qkv + row * 3 * A + which * A + (long long)h * D;
  const float* g = dqk + row * 2 * A + which * A + (long long)h * D;
  float y1[PER], y2[PER], g1[PER], g2[PER], cs[PER], sn[PER], x1[PER], x2[PER], ss = 0.f, dot = 0.f;
  if constexpr (PER == 2) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 2 * lane));
    const float2 c2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + HALF + 2 * lane));
    const float2 cc = *reinterpret_cast<const float2*>(cosT + (long long)t * HALF + 2 * lane);
    const float2 sc = *reinterpret_cast<const float2*>(sinT + (long long)t * HALF + 2 * lane);
    const float2 ga = *reinterpret_cast<const float2*>(g + 2 * lane);
    const float2 gb = *reinterpret_cast<const float2*>(g + HALF + 2 * lane);
    x1[0] = a.x; x1[1] = a.y; x2[0] = c2.x; x2[1] = c2.y; cs[0] = cc.x; cs[1] = cc.y; sn[0] = sc.x; sn[1] = sc.y;
    g1[0] = ga.x; g1[1] = ga.y; g2[0] = gb.x; g2[1] = gb.y;
  } else {
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = lane * PER + e;
      x1[e] = __bfloat162float(src[i]); x2[e] = __bfloat162float(src[HALF + i]);
      cs[e] = cosT[(long long)t * HALF + i]; sn[e] = sinT[(long long)t * HALF + i];
      g1[e] = g[i]; g2[e] = g[HALF + i];
    }
  }
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    y1[e] = x1[e] * cs[e] + x2[e] * sn[e];
    y2[e] = -x1[e] * sn[e] + x2[e] * cs[e];
    ss += y1[e] * y1[e] + y2[e] * y2[e];
    dot += y1[e] * g1[e] + y2[e] * g2[e];
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss / D + kQkEps);
  const float m = dot * r * r / D;     // mean(dxhat * xhat) * r, with xhat = u r
  float o1[PER], o2[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const float du1 = r * (g1[e] - y1[e] * m), du2 = r * (g2[e] - y2[e] * m);
    o1[e] = du1 * cs[e] - du2 * sn[e];
    o2[e] = du1 * sn[e] + du2 * cs[e];
  }
  if constexpr (PER == 2) {
    *reinterpret_cast<__nv_bfloat162*>(out + 2 * lane) = __floats2bfloat162_rn(o1[0], o1[1]);
    *reinterpret_cast<__nv_bfloat162*>(out + HALF + 2 * lane) = __floats2bfloat162_rn(o2[0], o2[1]);
  } else {
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int i = lane * PER + e;
      out[i] = __float2bfloat16(o1[e]);
      out[HALF + i] = __float2bfloat16(o2[e]);
    }
  }
}

// head_dim 128 fast paths: eight lanes per head vector (16-byte accesses: elements [8 l, 8 l + 8) of the first half and
// their rotate-half partners in the second half), four head vectors per warp, reductions over the 8-lane group.
__device__ __forceinline__ void ld8_bf16(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 v = unpack_bf16(w[t]);
    f[2 * t] = v.x;
    f[2 * t + 1] = v.y;
  }
}
__device__ __forceinline__ void st8_bf16(__nv_bfloat16* p, const float* f) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void ld8_f32(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ float group8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

// Eight threads per (row, head); a thread takes its 16 elements of the query head and of the key head, which share the
// rotation tables, so that 64 bytes of loads per thread are in flight (with 32 the kernel sat at 0.7 of the copy rate).
__global__ void rope_qknorm_fwd128_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                                          const float* __restrict__ sinT, __nv_bfloat16* __restrict__ qk, long long M, int T, int H) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;     // (row, head)
  const int l8 = threadIdx.x & 7;
  const long long total = M * H;
  const bool live = item < total;
  const long long it = live ? item : total - 1;
  const int h = (int)(it % H);
  const long long row = it / H;
  const int t = (int)(row % T);
  const long long A = (long long)H * 128;
  const __nv_bfloat16* src = qkv + row * 3 * A + (long long)h * 128 + l8 * 8;
  float x1[2][8], x2[2][8], cs[8], sn[8];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    ld8_bf16(src + w * A, x1[w]);
    ld8_bf16(src + w * A + 64, x2[w]);
  }
  ld8_f32(cosT + (long long)t * 64 + l8 * 8, cs);
  ld8_f32(sinT + (long long)t * 64 + l8 * 8, sn);
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    float y1[8], y2[8];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      y1[e] = x1[w][e] * cs[e] + x2[w][e] * sn[e];
      y2[e] = -x1[w][e] * sn[e] + x2[w][e] * cs[e];
      ss += y1[e] * y1[e] + y2[e] * y2[e];
    }
    ss = group8_sum(ss);
    const float r = rsqrtf(ss * (1.0f / 128.0f) + kQkEps);
#pragma unroll
    for (int e = 0; e < 8; ++e) { y1[e] *= r; y2[e] *= r; }
    if (live) {
      __nv_bfloat16* dst = qk + row * 2 * A + w * A + (long long)h * 128 + l8 * 8;
      st8_bf16(dst, y1);
      st8_bf16(dst + 64, y2);
    }
  }
}

__global__ void rope_qknorm_bwd128_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                                          const float* __restrict__ sinT, const float* __restrict__ dqk,
                                          const __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ dqkv, long long M, int T,
                                          int H) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;     // (row, q|k|v, head)
  const int l8 = threadIdx.x & 7;
  const long long total = M * 3 * H;
  const bool live = item < total;
  const long long it = live ? item : total - 1;
  const int h = (int)(it % H), which = (int)((it / H) % 3);
  const long long row = it / (3 * H);
  const long long A = (long long)H * 128;
  __nv_bfloat16* out = dqkv + row * 3 * A + which * A + (long long)h * 128 + l8 * 8;
  // `which` is uniform over each 8-lane group but may differ inside a warp; the shuffles below are executed by all lanes
  const int t = (int)(row % T);
  const bool is_v = which == 2;
  const int wq = is_v ? 0 : which;
  const __nv_bfloat16* src = qkv + row * 3 * A + wq * A + (long long)h * 128 + l8 * 8;
  const float* g = dqk + row * 2 * A + wq * A + (long long)h * 128 + l8 * 8;
  float x1[8], x2[8], cs[8], sn[8], g1[8], g2[8], y1[8], y2[8];
  ld8_bf16(src, x1);
  ld8_bf16(src + 64, x2);
  ld8_f32(cosT + (long long)t * 64 + l8 * 8, cs);
  ld8_f32(sinT + (long long)t * 64 + l8 * 8, sn);
  ld8_f32(g, g1);
  ld8_f32(g + 64, g2);
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    y1[e] = x1[e] * cs[e] + x2[e] * sn[e];
    y2[e] = -x1[e] * sn[e] + x2[e] * cs[e];
    ss += y1[e] * y1[e] + y2[e] * y2[e];
    dot += y1[e] * g1[e] + y2[e] * g2[e];
  }
  ss = group8_sum(ss);
  dot = group8_sum(dot);
  const float r = rsqrtf(ss * (1.0f / 128.0f) + kQkEps);
  const float m = dot * r * r * (1.0f / 128.0f);
  float o1[8], o2[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float du1 = r * (g1[e] - y1[e] * m), du2 = r * (g2[e] - y2[e] * m);
    o1[e] = du1 * cs[e] - du2 * sn[e];
    o2[e] = du1 * sn[e] + du2 * cs[e];
  }
  if (!live) return;
  if (is_v) {
    const __nv_bfloat16* gv = dv + row * A + (long long)h * 128 + l8 * 8;
    *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(gv);
    *reinterpret_cast<uint4*>(out + 64) = *reinterpret_cast<const uint4*>(gv + 64);
  } else {
    st8_bf16(out, o1);
    st8_bf16(out + 64, o2);
  }
}

// Same backward for bf16 dq-hat | dk-hat (the two-kernel attention backward writes them in bf16 and puts dV straight into
// its third of dqkv): only the q and k thirds are produced here.
__global__ void rope_qknorm_bwd128_bf16_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                                               const float* __restrict__ sinT, const __nv_bfloat16* __restrict__ dqk,
                                               __nv_bfloat16* __restrict__ dqkv, long long M, int T, int H) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;     // (row, head): query and key head
  const int l8 = threadIdx.x & 7;
  const long long total = M * H;
  const bool live = item < total;
  const long long it = live ? item : total - 1;
  const int h = (int)(it % H);
  const long long row = it / H;
  const long long A = (long long)H * 128;
  const long long col = (long long)h * 128 + l8 * 8;
  const __nv_bfloat16* src = qkv + row * 3 * A + col;
  const __nv_bfloat16* g = dqk + row * 2 * A + col;
  const int t = (int)(row % T);
  float x1[2][8], x2[2][8], g1[2][8], g2[2][8], cs[8], sn[8];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    ld8_bf16(src + w * A, x1[w]);
    ld8_bf16(src + w * A + 64, x2[w]);
    ld8_bf16(g + w * A, g1[w]);
    ld8_bf16(g + w * A + 64, g2[w]);
  }
  ld8_f32(cosT + (long long)t * 64 + l8 * 8, cs);
  ld8_f32(sinT + (long long)t * 64 + l8 * 8, sn);
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    float y1[8], y2[8];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      y1[e] = x1[w][e] * cs[e] + x2[w][e] * sn[e];
      y2[e] = -x1[w][e] * sn[e] + x2[w][e] * cs[e];
      ss += y1[e] * y1[e] + y2[e] * y2[e];
      dot += y1[e] * g1[w][e] + y2[e] * g2[w][e];
    }
    ss = group8_sum(ss);
    dot = group8_sum(dot);
    const float r = rsqrtf(ss * (1.0f / 128.0f) + kQkEps);
    const float m = dot * r * r * (1.0f / 128.0f);
    float o1[8], o2[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float du1 = r * (g1[w][e] - y1[e] * m), du2 = r * (g2[w][e] - y2[e] * m);
      o1[e] = du1 * cs[e] - du2 * sn[e];
      o2[e] = du1 * sn[e] + du2 * cs[e];
    }
    if (live) {
      __nv_bfloat16* out = dqkv + row * 3 * A + w * A + col;
      st8_bf16(out, o1);
      st8_bf16(out + 64, o2);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// forward attention, head_dim 128
// ---------------------------------------------------------------------------------------------------------------
struct AttnParams {
  int B, T, H;
  float c1;          // scale * log2(e)
  float c2;          // scale * D * log2(e)   (fixed softmax shift, in base-2 units)
  float shift_ln;    // scale * D
  int window_tiles;  // 0: full causal
  const int* doc_start;
  __nv_bfloat16* y;  // [B*T, H*128]
  float* lse;        // [B, H, T]
  int* err;
  int* items;        // device counter the persistent CTAs draw their work items from (zero at launch)
};

constexpr int AT = 128;                    // tile edge (queries and keys)
constexpr int AD = 128;                    // head dim
constexpr uint32_t TILE_BYTES = AT * AD * 2;   // 32 KB: two 128-byte-swizzled atoms of [128 rows][64 cols]
constexpr uint32_t ATOM_BYTES = TILE_BYTES / 2;

__device__ __forceinline__ int attn_first_tile(const AttnParams& p, int b, int qt) {
  int lo = 0;
  if (p.doc_start) lo = p.doc_start[(long long)b * p.T + qt * AT] / AT;
  if (p.window_tiles > 0) lo = max(lo, qt - p.window_tiles + 1);
  return lo;
}

// Persistent forward: one CTA per SM walks (query tile, head, batch) items.  Consecutive items are the query tiles of one
// (head, batch), so the CTAs that run at one time share their K/V tiles through L2 (dealing the heaviest tiles of all
// heads first made every CTA stream its own K/V from DRAM at once); the tile order is rotated from one (head, batch) to
// the next so that every CTA sees a mix of lengths.  All barrier phases run on across items: the producer loads the next
// item's Q and K/V while the current item computes, the MMA thread issues the next item's first S tiles while the softmax
// warps finish the current one, and the output accumulator is double-buffered in TMEM so the drain of item i happens
// after the first softmax tile of item i+1.
//   TMEM: S/P buffers at columns 0 and 128 (by running tile count), O buffers at 256 and 384 (by item parity).
//   smem: Q x 2 (item parity), K x 2 and V x 3 stages (running tile count): a K stage is free again once its S tile is
//   done, a V stage only after its O MMAs, so K and V rings of different depth keep the loads a full tile ahead.
__device__ int g_fwd_items;      // item counter of the persistent forward (one launch at a time per device)

struct FwdItem {
  int qt, h, b, kt0, n;
};
__device__ __forceinline__ FwdItem fwd_item(const AttnParams& p, int w, int n_tiles) {
  FwdItem it;
  const int grp = w / n_tiles;
  it.qt = n_tiles - 1 - (w % n_tiles + grp) % n_tiles;
  it.h = grp % p.H;
  it.b = grp / p.H;
  it.kt0 = attn_first_tile(p, it.b, it.qt);
  it.n = it.qt - it.kt0 + 1;
  return it;
}

// Threads: producer warp, MMA warp and sixteen softmax warps (four per 32-lane TMEM quadrant, 32 keys a thread).
constexpr int FWD_SW = 16;
constexpr uint32_t FWD_SLACK = 768;           // room for aligning the tiles to 1024 bytes (the seven tiles, the barriers and
                                             // the scratch fill the rest of the 227 KB)
constexpr int FWD_THREADS = 64 + 32 * FWD_SW;

__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qk, const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  if (base - raw > FWD_SLACK) {                       // the tiles would not fit behind the alignment gap
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_WAIT_AUX);
    return;
  }
  uint8_t* gen = smem_raw + (base - raw);
  auto sQ = [&](int s) { return base + TILE_BYTES * s; };
  auto sK = [&](int s) { return base + TILE_BYTES * (2 + s); };
  auto sV = [&](int s) { return base + TILE_BYTES * (4 + s); };
  constexpr uint32_t kBars = TILE_BYTES * 7;
  const uint32_t bars = base + kBars;
  auto q_full = [&](int s) { return bars + 8u * (0 + s); };
  auto q_free = [&](int s) { return bars + 8u * (2 + s); };
  auto k_full = [&](int s) { return bars + 8u * (4 + s); };
  auto k_free = [&](int s) { return bars + 8u * (6 + s); };
  auto v_full = [&](int s) { return bars + 8u * (8 + s); };
  auto v_free = [&](int s) { return bars + 8u * (11 + s); };
  auto s_full = [&](int s) { return bars + 8u * (14 + s); };
  auto p_full = [&](int s) { return bars + 8u * (16 + s); };
  auto o_full = [&](int s) { return bars + 8u * (18 + s); };
  auto o_free = [&](int s) { return bars + 8u * (20 + s); };
  const uint32_t tmem_slot = bars + 8u * 22;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + kBars + 176);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + kBars + 184);
  float* lsum = reinterpret_cast<float*>(gen + kBars + 256);           // [4 column parts][128 rows]
  const uint32_t ring_bars = bars + 192u;
  volatile int* ring_slots = reinterpret_cast<volatile int*>(gen + kBars + 224);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = p.H * AD;
  const int n_tiles = p.T / AT;
  const int total = n_tiles * p.H * p.B;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_free(s), 1);
      mbar_init(k_full(s), 1);
      mbar_init(k_free(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(p_full(s), FWD_SW);
      mbar_init(o_full(s), 1);
      mbar_init(o_free(s), FWD_SW);
    }
    for (int s = 0; s < 3; ++s) {
      mbar_init(v_full(s), 1);
      mbar_init(v_free(s), 1);
    }
    for (int s = 0; s < 4; ++s) mbar_init(ring_bars + 8u * s, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_qk);
    tma_prefetch_desc(&tm_v);
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
  auto tS = [&](int s) { return tmem + (uint32_t)s * 128u; };
  auto tO = [&](int s) { return tmem + 256u + (uint32_t)s * 128u; };

  // The producer and MMA roles run on all 32 lanes of their warp with warp-uniform state and issue from the elected lane
  // (`elect_one` in common.cuh: operands computed under a `lane == 0` branch cost about 80 clocks per `tcgen05.mma`, more
  // than the 64 clocks a 128 x 128 x 16 MMA executes).  Work items are drawn by lane 0 and handed round with a shuffle.
  // A lane whose bounded wait ran out turns `dead`: it walks on without waiting or issuing; when lane 0 is dead no
  // further item is drawn and the warp leaves together.
  if (warp == 0) {
    int g = 0, it = 0;
    bool dead = false;
    for (;; ++it) {
      int w = -1;
      if (lane == 0 && !dead) w = item_publish(ring_bars, ring_slots, it, p.items, total);
      w = warp_uniform(w);
      if (w < 0) break;
      FwdItem im = fwd_item(p, w, n_tiles);
      im.kt0 = warp_uniform(im.kt0);
      im.n = im.qt - im.kt0 + 1;
      const int qb = it & 1, row0 = im.b * p.T;
      if (it >= 2 && !dead) dead = !mbar_wait(q_free(qb), (uint32_t)(((it - 2) >> 1) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
      if (elect_one() && !dead) {
        mbar_arrive_expect_tx(q_full(qb), TILE_BYTES);
        tma_load_2d(sQ(qb), &tm_qk, q_full(qb), im.h * AD, row0 + im.qt * AT);
        tma_load_2d(sQ(qb) + ATOM_BYTES, &tm_qk, q_full(qb), im.h * AD + 64, row0 + im.qt * AT);
      }
      for (int j = 0; j < im.n; ++j, ++g) {
        const int ks = g & 1, vs = g % 3;
        const int r = row0 + (im.kt0 + j) * AT;
        if (g >= 2 && !dead) dead = !mbar_wait(k_free(ks), (uint32_t)(((g - 2) >> 1) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(k_full(ks), TILE_BYTES);
          tma_load_2d(sK(ks), &tm_qk, k_full(ks), A + im.h * AD, r);
          tma_load_2d(sK(ks) + ATOM_BYTES, &tm_qk, k_full(ks), A + im.h * AD + 64, r);
        }
        if (g >= 3 && !dead) dead = !mbar_wait(v_free(vs), (uint32_t)(((g - 3) / 3) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(v_full(vs), TILE_BYTES);
          tma_load_2d(sV(vs), &tm_v, v_full(vs), 2 * A + im.h * AD, r);
          tma_load_2d(sV(vs) + ATOM_BYTES, &tm_v, v_full(vs), 2 * A + im.h * AD + 64, r);
        }
      }
    }
  } else if (warp == 1) {
    const uint32_t idesc_s = umma_idesc_f16(128, 128, 1, 0, 0);   // Q (K-major) x K (K-major)
    const uint32_t idesc_o = umma_idesc_f16(128, 128, 1, 0, 1);   // P (TMEM) x V (MN-major)
    // the O += P V step of a tile is issued one tile late, behind the next tile's S, so the softmax of tile g runs
    // under the S MMAs of tile g+1.  P(g) sits in TMEM as packed bf16 pairs over the S(g) columns it was computed
    // from (each softmax warp packs its 32 columns into the first 16 of its own range).
    int pg = -1, p_item = 0;
    bool p_first = false, p_last = false, dead = false;
    auto issue_pv = [&]() {
      const int sb = pg & 1, ob = p_item & 1, vs = pg % 3;
      if (!dead) dead = !mbar_wait(v_full(vs), (uint32_t)((pg / 3) & 1), abort_flag, p.err, ERR_WAIT_FULL);
      if (!dead) dead = !mbar_wait(p_full(sb), (uint32_t)((pg >> 1) & 1), abort_flag, p.err, ERR_WAIT_AUX);
      if (p_first && p_item >= 2 && !dead)
        dead = !mbar_wait(o_free(ob), (uint32_t)(((p_item - 2) >> 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
      tc_fence_after();
      const uint64_t vdesc0 = umma_smem_desc(sV(vs), ATOM_BYTES, 1024, kLayoutSw128);     // + a compile-time step per UMMA_K
      if (elect_one() && !dead) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t bd = vdesc0 + (uint64_t)((k * 2048) >> 4);
          umma_f16_ts(tO(ob), tS(sb) + (uint32_t)((k >> 1) * 32 + (k & 1) * 8), bd, idesc_o, (p_first && k == 0) ? 0u : 1u);
        }
        tc_commit(v_free(vs));
        if (p_last) tc_commit(o_full(ob));
      }
    };
    int g = 0, it = 0;
    for (;; ++it) {
      int w = -1;
      if (!dead) w = item_take(ring_bars, ring_slots, it, abort_flag, p.err);
      w = warp_uniform(w);
      if (w < 0) break;
      FwdItem im = fwd_item(p, w, n_tiles);
      im.kt0 = warp_uniform(im.kt0);
      im.n = im.qt - im.kt0 + 1;
      const int qb = it & 1;
      if (!dead) dead = !mbar_wait(q_full(qb), (uint32_t)((it >> 1) & 1), abort_flag, p.err, ERR_WAIT_FULL);
      for (int j = 0; j < im.n; ++j, ++g) {
        const int sb = g & 1;
        if (!dead) dead = !mbar_wait(k_full(sb), (uint32_t)((g >> 1) & 1), abort_flag, p.err, ERR_WAIT_FULL);
        tc_fence_after();
        // S(g) overwrites the buffer that held P(g-2): its O MMAs were issued earlier on the same (in-order) pipe
        const uint64_t qdesc0 = umma_smem_desc(sQ(qb), 0, 1024, kLayoutSw128), kdesc0 = umma_smem_desc(sK(sb), 0, 1024, kLayoutSw128);
        if (elect_one() && !dead) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t off = (uint64_t)(((k >> 2) * ATOM_BYTES + (k & 3) * 32) >> 4);
            umma_f16(tS(sb), qdesc0 + off, kdesc0 + off, idesc_s, k ? 1u : 0u);
          }
          tc_commit(s_full(sb));
          tc_commit(k_free(sb));
          if (j == im.n - 1) tc_commit(q_free(qb));
        }
        if (pg >= 0) issue_pv();
        pg = g; p_item = it; p_first = j == 0; p_last = j == im.n - 1;
      }
    }
    if (pg >= 0) issue_pv();
  } else {
    // Softmax: sixteen warps, four per 32-lane TMEM quadrant; each thread owns one query row and 32 of the tile's 128
    // keys.  A tile's softmax is a chain -- TMEM load, exponentials, TMEM store -- that every warp runs at the same
    // time; with eight warps and 64 keys a thread a tile took 2 400 clocks against 1 024 of MMAs, sixteen warps take a
    // little less (0.207 -> 0.196 ms at B = 16, T = 2048, H = 10).  Two groups of eight warps that take alternate key
    // tiles (each chain then has two tile periods) were measured as well and were no faster (0.204 ms): with 64 keys a
    // thread the chain itself is twice as long.
    const int q = warp & 3, part = (warp - 2) >> 2;
    const int r = q * 32 + lane;            // row within the tile == TMEM lane
    const int c0 = part * 32;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    // the drain of an item's output is deferred until the first tile of the next item has been exponentiated
    bool pend = false, ok = true;
    int pend_it = 0;
    float pend_inv = 0.f;
    __nv_bfloat16* pend_y = nullptr;
    auto drain = [&]() -> bool {
      const int ob = pend_it & 1;
      const bool got = mbar_wait(o_full(ob), (uint32_t)((pend_it >> 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) return false;
      tc_fence_after();
      {
        uint32_t v[32];
        __syncwarp();
        BONES_TMEM_LD32(tO(ob) + lane_addr + (uint32_t)c0, v);
        tmem_ld_wait();
        uint4 u[4];
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          u[gq].x = pack_bf16(__uint_as_float(v[gq * 8 + 0]) * pend_inv, __uint_as_float(v[gq * 8 + 1]) * pend_inv);
          u[gq].y = pack_bf16(__uint_as_float(v[gq * 8 + 2]) * pend_inv, __uint_as_float(v[gq * 8 + 3]) * pend_inv);
          u[gq].z = pack_bf16(__uint_as_float(v[gq * 8 + 4]) * pend_inv, __uint_as_float(v[gq * 8 + 5]) * pend_inv);
          u[gq].w = pack_bf16(__uint_as_float(v[gq * 8 + 6]) * pend_inv, __uint_as_float(v[gq * 8 + 7]) * pend_inv);
        }
        st_global_v8(pend_y, u[0], u[1]);                // one full 32-byte sector per store
        st_global_v8(pend_y + 16, u[2], u[3]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free(ob));
      pend = false;
      return true;
    };
    int g = 0, it = 0;
    for (;; ++it) {
      const int w = ok ? item_take(ring_bars, ring_slots, it, abort_flag, p.err) : -1;
      if (w < 0) break;
      const FwdItem im = fwd_item(p, w, n_tiles);
      const int qpos = im.qt * AT + r, row0 = im.b * p.T;
      int lo = 0;
      if (p.doc_start) lo = p.doc_start[(long long)im.b * p.T + qpos];
      float l = 0.f;
      for (int j = 0; j < im.n; ++j, ++g) {
        const int sb = g & 1;
        const bool got = mbar_wait(s_full(sb), (uint32_t)((g >> 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        const int k0 = (im.kt0 + j) * AT + c0;
        // warp-uniform: does any row of this warp need the element mask for these 32 keys (diagonal or document start)?
        const bool need_mask = __any_sync(0xffffffffu, (k0 + 31 > qpos) || (k0 < lo));
        uint32_t v0[32], pk[16];
        __syncwarp();
        BONES_TMEM_LD32(tS(sb) + lane_addr + (uint32_t)c0, v0);
        tmem_ld_wait();
        {
          float e[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = fmaf(__uint_as_float(v0[i]), p.c1, -p.c2);
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e[i]) : "f"(x));
          }
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kpos = k0 + i;
              if (kpos > qpos || kpos < lo) e[i] = 0.f;
            }
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) l += e[i];
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(e[2 * i], e[2 * i + 1]);
        }
        BONES_TMEM_ST16(tS(sb) + lane_addr + (uint32_t)c0, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(sb));
        if (pend && !drain()) { ok = false; break; }
      }
      if (!ok) break;
      // the four threads of a row exchange their partial row sums through shared memory
      lsum[part * AT + r] = l;
      asm volatile("bar.sync 1, 512;" ::: "memory");
      l = (lsum[r] + lsum[AT + r]) + (lsum[2 * AT + r] + lsum[3 * AT + r]);      // the same order in all four threads
      asm volatile("bar.sync 1, 512;" ::: "memory");      // nobody rewrites the scratch before everybody has read it
      if (part == 0) p.lse[((long long)im.b * p.H + im.h) * p.T + qpos] = logf(l) + p.shift_ln;
      pend = true;
      pend_it = it;
      pend_inv = 1.0f / l;
      pend_y = p.y + ((long long)(row0 + qpos)) * A + (long long)im.h * AD + c0;
    }
    if (ok && pend) drain();
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

static int tmap_rows_2d(CUtensorMap* out, const void* ptr, long long rows, long long cols) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)cols * 2};
  uint32_t box[2] = {64, 128};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace bones

extern "C" {
using namespace bones;

int bones_rope_qknorm_fwd(const void* qkv, const float* cosT, const float* sinT, void* qk, long long M, int T, int H, int D, void* stream) {
  const long long warps = M * H * 2;
  const unsigned grid = (unsigned)((warps + 7) / 8);
  if (D == 128) {
    const long long threads = M * H * 8;
    rope_qknorm_fwd128_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)qkv, cosT, sinT,
                                                                                                   (__nv_bfloat16*)qk, M, T, H);
  }
  else if (D == 64)
    rope_qknorm_fwd_kernel<64><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)qkv, cosT, sinT, (__nv_bfloat16*)qk, M, T, H);
  else
    return -2;
  return (int)cudaGetLastError();
}

int bones_rope_qknorm_bwd(const void* qkv, const float* cosT, const float* sinT, const float* dqk, const void* dv, void* dqkv, long long M,
                          int T, int H, int D, void* stream) {
  const long long warps = M * H * 3;
  const unsigned grid = (unsigned)((warps + 7) / 8);
  if (D == 128) {
    const long long threads = M * 3 * H * 8;
    rope_qknorm_bwd128_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)qkv, cosT, sinT, dqk, (const __nv_bfloat16*)dv, (__nv_bfloat16*)dqkv, M, T, H);
  }
  else if (D == 64)
    rope_qknorm_bwd_kernel<64><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)qkv, cosT, sinT, dqk, (const __nv_bfloat16*)dv,
                                                                    (__nv_bfloat16*)dqkv, M, T, H);
  else
    return -2;
  return (int)cudaGetLastError();
}

// dqk: bf16 [M, 2*H*128]; writes the q and k thirds of dqkv [M, 3*H*128] (head_dim 128 only)
int bones_rope_qknorm_bwd_bf16(const void* qkv, const float* cosT, const float* sinT, const void* dqk, void* dqkv, long long M, int T, int H,
                               void* stream) {
  const long long threads = M * H * 8;
  rope_qknorm_bwd128_bf16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, cosT, sinT, (const __nv_bfloat16*)dqk, (__nv_bfloat16*)dqkv, M, T, H);
  return (int)cudaGetLastError();
}

// qk: [B*T, 2*H*128] (rotated, normalised q and k); qkv: [B*T, 3*H*128] (values read in place); y: [B*T, H*128]; lse: [B,H,T]
int bones_attn_fwd(const void* qk, const void* qkv, void* y, float* lse, const int* doc_start, int B, int T, int H, float scale,
                   int window_tiles, void* stream) {
  if (T % AT) return -2;
  CUtensorMap tq, tv;
  const long long M = (long long)B * T, A = (long long)H * AD;
  int rc = tmap_rows_2d(&tq, qk, M, 2 * A);
  if (rc) return rc;
  rc = tmap_rows_2d(&tv, qkv, M, 3 * A);
  if (rc) return rc;
  AttnParams p;
  p.B = B; p.T = T; p.H = H;
  p.c1 = scale * 1.4426950408889634f;
  p.c2 = scale * AD * 1.4426950408889634f;
  p.shift_ln = scale * AD;
  p.window_tiles = window_tiles;
  p.doc_start = doc_start;
  p.y = (__nv_bfloat16*)y;
  p.lse = lse;
  p.err = error_word();
  constexpr size_t smem = (size_t)TILE_BYTES * 7 + 256 + 2048 + FWD_SLACK;   // tiles, barriers, row-sum scratch, alignment slack
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const long long items = (long long)(T / AT) * H * B;
  const unsigned grid = (unsigned)(items < sms ? items : sms);       // persistent: one CTA per SM
  static int* counter[64] = {};
  if (dev < 0 || dev >= 64) return -2;
  if (!counter[dev]) BONES_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&counter[dev]), g_fwd_items));
  BONES_CHECK(cudaMemsetAsync(counter[dev], 0, sizeof(int), (cudaStream_t)stream));
  p.items = counter[dev];
  attn_fwd_kernel<<<grid, FWD_THREADS, smem, (cudaStream_t)stream>>>(tq, tv, p);
  return (int)cudaGetLastError();
}
}  // extern "C"
