// Fused compute + collective kernels over NVLink peer memory (no NCCL call on these paths).
//
// Every rank maps every other rank's slabs (symmetric allocations; the host exchanges the peer pointers once).  A kernel
// on rank r then reads its owned chunk straight out of all W gradient slabs with peer loads, reduces in registers and
// feeds the optimizer math in the same pass; updated low-precision shards are stored straight into all W weight slabs
// with peer stores.  Replaces, for the data-parallel optimizer step, reduce_scatter_tensor + elementwise kernels +
// all_gather_into_tensor (reference call sites: round2/source/train.py:13136-13160 reduce-scatter, :13211-13247
// updates + all-gather, :13183-13186 scalar all-reduce).
//
// Cross-GPU ordering uses epoch flags in symmetric memory: a rank publishes `epoch` into its slot on every peer with a
// system-scope release store after its own work is visible, and waits with system-scope acquire loads until every
// peer's slot in its own flag array has reached the epoch.  Waits are bounded: on expiry the kernel records
// ERR_WAIT_PEER in the error word and returns, and the host raises.  Plain peer loads/stores only: no multimem, so a
// rank that has left cannot fault the others.
#include "common.cuh"

namespace bones {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* addr) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(addr) : "memory");
  return v;
}

// All-rank barrier: flags[rank][slot j] lives on `rank`; rank r writes its epoch into slot r of every peer, then waits for
// all slots of its own array.  The epoch is a device-side counter of this rank that the kernel itself advances (every
// rank runs the same sequence of barriers, so the counters agree): nothing about a barrier is baked into its launch
// arguments, and a CUDA graph that contains barriers can be replayed.  One block; thread j handles peer j.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int* epoch_dev, long long limit_cycles, int* err) {
  __shared__ int epoch_s;
  const int j = threadIdx.x;
  if (j == 0) epoch_s = *epoch_dev + 1;
  __syncthreads();
  const int epoch = epoch_s;
  __threadfence_system();
  if (j < world) st_release_sys(reinterpret_cast<int*>(flags.p[j]) + rank, epoch);
  if (j < world) {
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + j;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > limit_cycles) {
        atomicCAS(err, 0, ERR_WAIT_PEER);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (j == 0) *epoch_dev = epoch;
}

// Sum of W fp32 vectors, identical on every rank (small scalar stacks): out[i] = scale * sum_r in_r[i].
__global__ void peer_allreduce_small_kernel(PeerPtrs in, float* out, int n, int world, float scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int r = 0; r < world; ++r) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(reinterpret_cast<const float*>(in.p[r]) + i) : "memory");
    s += v;
  }
  out[i] = s * scale;
}

// NVSwitch multicast (NVLS): one load from the multicast address of a symmetric buffer returns the sum of all ranks'
// copies, added inside the switch, so a reduction over W ranks moves one element over this GPU's links instead of W - 1;
// one store to the multicast address lands in every rank's copy.  `mc` pointers are null when the buffer has no
// multicast mapping (or BONES_NVLS=0): the kernels then loop over the peer pointers.
__device__ __forceinline__ float4 ld_multimem_sum_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_multimem_bf16x4(__nv_bfloat16* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(mc), "r"(v.x), "r"(v.y) : "memory");
}

// Reduce-scatter fused with the Muon prologue on the owned chunk [off, off + n):
//   g = scale * sum_r G_r[off + i];  m += (1 - mu) (g - m);  u = g + mu (m - g);  X = bf16(u);  sumsq[mat] += u^2
//   gsq += g^2 (finiteness gate)
__global__ void rs_muon_prep_kernel(PeerPtrs G, long long off, long long n, int world, float scale, float mu, float* __restrict__ mom,
                                    __nv_bfloat16* __restrict__ X, float* __restrict__ sumsq, long long mat_elems, float* __restrict__ gsq,
                                    const float* __restrict__ mcG) {
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  float local = 0.f, lg = 0.f;
  long long mat = 0;
  if (i4 < n) {
    float4 s = make_float4(0, 0, 0, 0);
    if (mcG) {
      s = ld_multimem_sum_f4(mcG + off + i4);
    } else {
      for (int r = 0; r < world; ++r) {
        const float4 v = ld_peer_f4(reinterpret_cast<const float*>(G.p[r]) + off + i4);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    lg = s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    // finiteness gate: a non-finite reduced gradient contributes nothing to the update (lg still records it)
    if (!isfinite(lg)) s = make_float4(isfinite(s.x) ? s.x : 0.f, isfinite(s.y) ? s.y : 0.f, isfinite(s.z) ? s.z : 0.f,
                                       isfinite(s.w) ? s.w : 0.f);
    float4 m = *reinterpret_cast<float4*>(mom + i4);
    m.x += (1.f - mu) * (s.x - m.x); m.y += (1.f - mu) * (s.y - m.y);
    m.z += (1.f - mu) * (s.z - m.z); m.w += (1.f - mu) * (s.w - m.w);
    *reinterpret_cast<float4*>(mom + i4) = m;
    const float u0 = s.x + mu * (m.x - s.x), u1 = s.y + mu * (m.y - s.y), u2 = s.z + mu * (m.z - s.z), u3 = s.w + mu * (m.w - s.w);
    const __nv_bfloat162 b0 = __floats2bfloat162_rn(u0, u1), b1 = __floats2bfloat162_rn(u2, u3);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&b0);
    o.y = *reinterpret_cast<const uint32_t*>(&b1);
    *reinterpret_cast<uint2*>(X + i4) = o;
    const float2 f0 = __bfloat1622float2(b0), f1 = __bfloat1622float2(b1);   // the norm of what the iteration will see
    local = f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
    mat = i4 / mat_elems;
  }
  // a block never straddles a matrix when mat_elems is a multiple of blockDim.x * 4 (checked on the host)
  __shared__ float red[2][32];
  local = warp_sum(local);
  lg = warp_sum(lg);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = local; red[1][threadIdx.x >> 5] = lg; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    float a = threadIdx.x < nw ? red[0][threadIdx.x] : 0.f, b = threadIdx.x < nw ? red[1][threadIdx.x] : 0.f;
    a = warp_sum(a);
    b = warp_sum(b);
    if (threadIdx.x == 0) {
      const long long first = (long long)blockIdx.x * blockDim.x * 4;
      if (first < n) {
        atomicAdd(sumsq + first / mat_elems, a);
        atomicAdd(gsq, b);
      }
    }
  }
  (void)mat;
}

// X[mat] *= 1 / (sqrt(sumsq[mat]) * 1.01 + 1e-6)   (Frobenius normalisation before Newton-Schulz)
__global__ void muon_normalize_kernel(__nv_bfloat16* X, const float* sumsq, long long n, long long mat_elems) {
  const long long i2 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i2 >= n) return;
  const float inv = 1.0f / (sqrtf(sumsq[i2 / mat_elems]) * 1.01f + 1e-6f);
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(X + i2);
  const float2 f = __bfloat1622float2(*p);
  *p = __floats2bfloat162_rn(f.x * inv, f.y * inv);
}

// Reduce-scatter + AdamW + publish in one pass over the owned rows [off, off + n):
//   g = scale * sum_r G_r[off + i]; AdamW on (master, m, v); bf16(master) stored into every rank's weight slab at off + i.
__global__ void rs_adamw_publish_kernel(PeerPtrs G, PeerPtrs Wt, long long off, long long n, int world, float scale, float* __restrict__ master,
                                        float* __restrict__ m1, float* __restrict__ m2, float lr, float b1, float b2, float eps, float wd,
                                        float c1, float c2, float* __restrict__ gsq, const float* __restrict__ mcG,
                                        __nv_bfloat16* __restrict__ mcW) {
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  float lg = 0.f;
  if (i4 < n) {
    float4 s = make_float4(0, 0, 0, 0);
    if (mcG) {
      s = ld_multimem_sum_f4(mcG + off + i4);
    } else {
      for (int r = 0; r < world; ++r) {
        const float4 v = ld_peer_f4(reinterpret_cast<const float*>(G.p[r]) + off + i4);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
    }
    float g[4] = {s.x * scale, s.y * scale, s.z * scale, s.w * scale};
    float4 p = *reinterpret_cast<float4*>(master + i4), a = *reinterpret_cast<float4*>(m1 + i4), b = *reinterpret_cast<float4*>(m2 + i4);
    float pp[4] = {p.x, p.y, p.z, p.w}, aa[4] = {a.x, a.y, a.z, a.w}, bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      lg += g[t] * g[t];
      if (!isfinite(g[t])) g[t] = 0.f;       // finiteness gate (lg keeps the evidence)
      pp[t] *= 1.0f - lr * wd;
      aa[t] += (1.0f - b1) * (g[t] - aa[t]);
      bb[t] += (1.0f - b2) * (g[t] * g[t] - bb[t]);
      pp[t] -= lr * (aa[t] / c1) / (sqrtf(bb[t] / c2) + eps);
    }
    *reinterpret_cast<float4*>(master + i4) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    *reinterpret_cast<float4*>(m1 + i4) = make_float4(aa[0], aa[1], aa[2], aa[3]);
    *reinterpret_cast<float4*>(m2 + i4) = make_float4(bb[0], bb[1], bb[2], bb[3]);
    uint2 o;
    o.x = pack_bf16(pp[0], pp[1]);
    o.y = pack_bf16(pp[2], pp[3]);
    if (mcW) st_multimem_bf16x4(mcW + off + i4, o);
    else
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(Wt.p[r]) + off + i4) = o;
  }
  lg = warp_sum(lg);
  if ((threadIdx.x & 31) == 0 && !(lg == 0.f)) atomicAdd(gsq, lg);
}

// Publish: bf16(src[i]) stored into every rank's weight slab at off + i (src fp32 master of the owned chunk).
__global__ void peer_publish_kernel(const float* __restrict__ src, PeerPtrs Wt, long long off, long long n, int world,
                                    __nv_bfloat16* __restrict__ mcW) {
  const long long i4 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= n) return;
  const float4 v = *reinterpret_cast<const float4*>(src + i4);
  uint2 o;
  o.x = pack_bf16(v.x, v.y);
  o.y = pack_bf16(v.z, v.w);
  if (mcW) st_multimem_bf16x4(mcW + off + i4, o);
  else
    for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(Wt.p[r]) + off + i4) = o;
}

// MoE / table exchange helper: rows gathered from peers.  out[i] = table_{owner[i]}[local[i]] (bf16 rows of C columns).
__global__ void peer_gather_rows_kernel(PeerPtrs tables, const long long* __restrict__ ids, __nv_bfloat16* __restrict__ out, int n, int C,
                                        int world, long long rows_per_shard) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const long long id = ids[row];
  const int owner = (int)(id % world);
  const long long local = id / world;
  if (!BONES_INDEX_OK(local, 0, rows_per_shard)) return;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(tables.p[owner]) + local * C;
  for (int c = lane * 8; c < C; c += 256) {
    uint4 u;
    asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(src + c) : "memory");
    *reinterpret_cast<uint4*>(out + (size_t)row * C + c) = u;
  }
}

// Equal-split all-to-all by peer stores: chunk d of my `src` ([W, chunk] elements of 16 bytes) is written into slot
// `rank` of peer d's `dst` ([W, chunk]).
__global__ void peer_all_to_all_kernel(const uint4* __restrict__ src, PeerPtrs dst, long long chunk16, int rank, int world) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = chunk16 * world;
  if (i >= total) return;
  const int d = (int)(i / chunk16);
  const long long j = i - (long long)d * chunk16;
  reinterpret_cast<uint4*>(dst.p[d])[(long long)rank * chunk16 + j] = src[i];
}

// MoE dispatch fused with the expert-parallel exchange: slot s of the [E, b, C] slot buffer belongs to rank
// d = s / rows_per_dest; its token row h[tok[s]] (or zeros for an empty slot) is stored straight into rank d's receive
// buffer at [source rank][s % rows_per_dest]: the permute and the all-to-all are one pass over NVLink, and no local slot
// buffer exists.  One warp per slot.
__global__ void peer_dispatch_rows_kernel(const __nv_bfloat16* __restrict__ h, const long long* __restrict__ tok, PeerPtrs dst,
                                          long long rows_per_dest, long long n_slots, long long n_tokens, int C, int rank) {
  const long long s = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (s >= n_slots) return;
  const int d = (int)(s / rows_per_dest);
  const long long j = s - (long long)d * rows_per_dest;
  const long long t = tok[s];
  const bool valid = t >= 0 && t < n_tokens;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(dst.p[d]) + ((long long)rank * rows_per_dest + j) * C;
  for (int c = lane * 8; c < C; c += 256) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (valid) u = *reinterpret_cast<const uint4*>(h + t * C + c);
    *reinterpret_cast<uint4*>(out + c) = u;
  }
}

// MoE dispatch written in the consumer's layout: slot s = (expert e, j) of the [E, rows] slot buffer (rows = b * C)
// belongs to rank d = e / m and lands there at [(e % m), source rank, j] of a [m, W, rows] buffer, which is exactly the
// [local expert][all ranks' rows] grouping the expert GEMMs read: no transposing copy after the exchange.
__global__ void peer_dispatch_grouped_kernel(const __nv_bfloat16* __restrict__ h, const long long* __restrict__ tok, PeerPtrs dst, long long rows,
                                             int m, long long n_slots, long long n_tokens, int C, int rank, int world) {
  const long long s = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (s >= n_slots) return;
  const long long e = s / rows, j = s - e * rows;
  const int d = (int)(e / m), el = (int)(e - (long long)d * m);
  const long long t = tok[s];
  (void)BONES_INDEX_OK(t, 0, n_tokens + 1);               // n_tokens itself marks an empty slot
  const bool valid = t >= 0 && t < n_tokens;
  if (!BONES_INDEX_OK(d, 0, world)) return;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(dst.p[d]) + (((long long)el * world + rank) * rows + j) * C;
  for (int c = lane * 8; c < C; c += 256) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (valid) u = *reinterpret_cast<const uint4*>(h + t * C + c);
    *reinterpret_cast<uint4*>(out + c) = u;
  }
}

// Block-permuting all-to-all between the two MoE layouts (blocks of `rows` rows of C bf16), by peer stores:
//   mode 0, to the experts:  source [W(dst), m, rows]  ->  on rank w: [m, W(src), rows]   block (w, e) -> (e, rank)
//   mode 1, to the sources:  source [m, W(dst), rows]  ->  on rank w: [W * m, rows]        block (e, w) -> (rank * m + e)
// One warp per row.
__global__ void peer_blocks_kernel(const __nv_bfloat16* __restrict__ src, PeerPtrs dst, long long rows, int m, int C, int rank, int world,
                                   int mode) {
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long long total = rows * m * world;
  if (r >= total) return;
  const long long blk = r / rows, j = r - blk * rows;
  int w, e;
  long long dblk;
  if (mode == 0) {
    w = (int)(blk / m); e = (int)(blk - (long long)w * m);
    dblk = (long long)e * world + rank;
  } else {
    e = (int)(blk / world); w = (int)(blk - (long long)e * world);
    dblk = (long long)rank * m + e;
  }
  const __nv_bfloat16* in = src + r * C;
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(dst.p[w]) + (dblk * rows + j) * C;
  for (int c = lane * 8; c < C; c += 256) *reinterpret_cast<uint4*>(out + c) = *reinterpret_cast<const uint4*>(in + c);
}

static PeerPtrs make_ptrs(void* const* ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < kMaxPeers; ++i) p.p[i] = i < world ? ptrs[i] : nullptr;
  return p;
}

}  // namespace bones

extern "C" {
using namespace bones;

int bones_peer_barrier(void* const* flag_ptrs, int rank, int world, int* epoch_dev, double limit_seconds, void* stream) {
  if (world > kMaxPeers) return -2;
  const long long limit = (long long)(limit_seconds * 1.9e9);
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_ptrs(flag_ptrs, world), rank, world, epoch_dev, limit, error_word());
  return (int)cudaGetLastError();
}

int bones_peer_allreduce_small(void* const* in_ptrs, float* out, int n, int world, float scale, void* stream) {
  if (world > kMaxPeers) return -2;
  peer_allreduce_small_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(make_ptrs(in_ptrs, world), out, n, world, scale);
  return (int)cudaGetLastError();
}

int bones_rs_muon_prep_mc(void* const* g_ptrs, long long off, long long n, int world, float scale, float mu, float* mom, void* X, float* sumsq,
                          long long mat_elems, float* gsq, const void* mc_g, void* stream) {
  if (world > kMaxPeers || (n % 4) || (off % 4) || (mat_elems % 1024) || ((uintptr_t)mc_g & 15)) return -2;
  const long long threads = n / 4;
  rs_muon_prep_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(make_ptrs(g_ptrs, world), off, n, world, scale, mu, mom,
                                                                                         (__nv_bfloat16*)X, sumsq, mat_elems, gsq,
                                                                                         (const float*)mc_g);
  return (int)cudaGetLastError();
}
int bones_rs_muon_prep(void* const* g_ptrs, long long off, long long n, int world, float scale, float mu, float* mom, void* X, float* sumsq,
                       long long mat_elems, float* gsq, void* stream) {
  return bones_rs_muon_prep_mc(g_ptrs, off, n, world, scale, mu, mom, X, sumsq, mat_elems, gsq, nullptr, stream);
}

int bones_muon_normalize(void* X, const float* sumsq, long long n, long long mat_elems, void* stream) {
  if ((n % 2) || (mat_elems % 2)) return -2;
  muon_normalize_kernel<<<(unsigned)((n / 2 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)X, sumsq, n, mat_elems);
  return (int)cudaGetLastError();
}

// mc_g / mc_w: multicast addresses of the gradient and weight slabs (null: peer loops)
int bones_rs_adamw_publish_mc(void* const* g_ptrs, void* const* w_ptrs, long long off, long long n, int world, float scale, float* master,
                              float* m1, float* m2, float lr, float b1, float b2, float eps, float wd, int step, float* gsq, const void* mc_g,
                              void* mc_w, void* stream) {
  if (world > kMaxPeers || (n % 4) || (off % 4) || ((uintptr_t)mc_g & 15) || ((uintptr_t)mc_w & 7)) return -2;
  const float c1 = 1.0f - powf(b1, (float)step), c2 = 1.0f - powf(b2, (float)step);
  rs_adamw_publish_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      make_ptrs(g_ptrs, world), make_ptrs(w_ptrs, world), off, n, world, scale, master, m1, m2, lr, b1, b2, eps, wd, c1, c2, gsq,
      (const float*)mc_g, (__nv_bfloat16*)mc_w);
  return (int)cudaGetLastError();
}
int bones_rs_adamw_publish(void* const* g_ptrs, void* const* w_ptrs, long long off, long long n, int world, float scale, float* master, float* m1,
                           float* m2, float lr, float b1, float b2, float eps, float wd, int step, float* gsq, void* stream) {
  return bones_rs_adamw_publish_mc(g_ptrs, w_ptrs, off, n, world, scale, master, m1, m2, lr, b1, b2, eps, wd, step, gsq, nullptr, nullptr, stream);
}

int bones_peer_publish_mc(const float* src, void* const* w_ptrs, long long off, long long n, int world, void* mc_w, void* stream) {
  if (world > kMaxPeers || (n % 4) || (off % 4) || ((uintptr_t)mc_w & 7)) return -2;
  peer_publish_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(src, make_ptrs(w_ptrs, world), off, n, world,
                                                                                       (__nv_bfloat16*)mc_w);
  return (int)cudaGetLastError();
}
int bones_peer_publish(const float* src, void* const* w_ptrs, long long off, long long n, int world, void* stream) {
  return bones_peer_publish_mc(src, w_ptrs, off, n, world, nullptr, stream);
}

int bones_peer_gather_rows(void* const* table_ptrs, const long long* ids, void* out, int n, int C, int world, long long rows_per_shard,
                           void* stream) {
  if (world > kMaxPeers || (C % 8)) return -2;
  peer_gather_rows_kernel<<<(n + 7) / 8, 256, 0, (cudaStream_t)stream>>>(make_ptrs(table_ptrs, world), ids, (__nv_bfloat16*)out, n, C, world,
                                                                         rows_per_shard);
  return (int)cudaGetLastError();
}

int bones_peer_dispatch_rows(const void* h, const long long* tok, void* const* dst_ptrs, long long rows_per_dest, long long n_slots,
                             long long n_tokens, int C, int rank, int world, void* stream) {
  if (world > kMaxPeers || (C % 8)) return -2;
  peer_dispatch_rows_kernel<<<(unsigned)((n_slots + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)h, tok, make_ptrs(dst_ptrs, world),
                                                                                           rows_per_dest, n_slots, n_tokens, C, rank);
  return (int)cudaGetLastError();
}

int bones_peer_dispatch_grouped(const void* h, const long long* tok, void* const* dst_ptrs, long long rows, int m, long long n_slots,
                                long long n_tokens, int C, int rank, int world, void* stream) {
  if (world > kMaxPeers || (C % 8)) return -2;
  peer_dispatch_grouped_kernel<<<(unsigned)((n_slots + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)h, tok, make_ptrs(dst_ptrs, world),
                                                                                              rows, m, n_slots, n_tokens, C, rank, world);
  return (int)cudaGetLastError();
}

int bones_peer_blocks(const void* src, void* const* dst_ptrs, long long rows, int m, int C, int rank, int world, int mode, void* stream) {
  if (world > kMaxPeers || (C % 8)) return -2;
  const long long total = rows * m * world;
  peer_blocks_kernel<<<(unsigned)((total + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, make_ptrs(dst_ptrs, world), rows, m, C,
                                                                                    rank, world, mode);
  return (int)cudaGetLastError();
}

int bones_peer_all_to_all(const void* src, void* const* dst_ptrs, long long chunk_bytes, int rank, int world, void* stream) {
  if (world > kMaxPeers || (chunk_bytes % 16)) return -2;
  const long long chunk16 = chunk_bytes / 16, total = chunk16 * world;
  peer_all_to_all_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)src, make_ptrs(dst_ptrs, world), chunk16,
                                                                                          rank, world);
  return (int)cudaGetLastError();
}
}  // extern "C"
BONES_BOUNDS_EXPORT(comm)
