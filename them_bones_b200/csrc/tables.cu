// Hashed n-gram tables, gradient side: sparse-gradient exchange over NVLink peer memory and the owner's sparse update,
// with no library collective, no host synchronisation and no dense gradient.
//
// Owner of global row r is rank r % W, its local index r / W.  Three kernels per table and step:
//
//   table_push      (every rank, during backward) one warp per (row id, gradient row): a system-scope atomic on the
//                   owner's entry counter reserves a slot in the owner's staging buffer, then the local row id and the
//                   bf16 gradient row are stored there with peer stores.  The permute-by-owner, the all-to-all and the
//                   count exchange of the library path are this one pass; the host never learns a count.
//   (epoch barrier, comm.cu; then a device-side sort of the staged ids: a key sort, no host round trip)
//   table_update    (owner) one warp per staged entry in sorted order; the warp that holds the first entry of a row
//                   sums the row's run of duplicates in registers, averages over the ranks and applies the optimizer to
//                   the bf16 table row in place.  Deterministic: no atomics on values, the sum runs in sorted order.
//   table_reset     (owner) staged ids back to the "empty" key, counter to zero.
//
// Optimizers: row-wise RMS (the reference's table update: one fp32 second moment per row,
// acc = beta acc + (1 - beta) mean(g^2); row = row (1 - decay) - lr g / (sqrt(acc) + eps), stochastic rounding to bf16;
// round2/source/train.py:3678-3701) or Adam with dense fp32 moments indexed by row.  A row whose summed gradient is not
// finite is skipped and counted (the reference skips the whole update; a per-row gate needs no host decision).
//
// Reference counterpart of the exchange: `_exchange` (owner = ids % W, staging slots in /dev/shm, barriers),
// round2/source/train.py:3653-3680.
#include "common.cuh"

namespace bones {

constexpr int kTabMaxPeers = 8;
struct TabPeers {
  void* p[kTabMaxPeers];
};
constexpr long long kEmptyKey = 0x7fffffffffffffffLL;

__device__ __forceinline__ uint32_t tab_hash(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t h = a * 0x9E3779B1u ^ (b + 0x7F4A7C15u) * 0x85EBCA6Bu ^ (c + 0x165667B1u) * 0xC2B2AE35u;
  h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
  return h;
}

__global__ void table_push_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ g, long long n, int C, TabPeers stage_ids,
                                  TabPeers stage_g, TabPeers stage_cnt, int cap, int world, int* __restrict__ overflow, long long rows_per_shard) {
  const long long e = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (e >= n) return;
  const long long id = ids[e];
  const int owner = (int)(id % world);
  const long long local = id / world;
  if (!BONES_INDEX_OK(local, 0, rows_per_shard)) return;
  int pos = 0;
  if (lane == 0) pos = atomicAdd_system(reinterpret_cast<int*>(stage_cnt.p[owner]), 1);
  pos = __shfl_sync(0xffffffffu, pos, 0);
  if (pos >= cap) {
    if (lane == 0) atomicAdd(overflow, 1);
    return;
  }
  if (lane == 0) reinterpret_cast<long long*>(stage_ids.p[owner])[pos] = local;
  const __nv_bfloat16* src = g + e * C;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(stage_g.p[owner]) + (long long)pos * C;
  for (int c = lane * 8; c < C; c += 256) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
}

// mode 0: row-wise RMS (state0 [rows] fp32).  mode 1: Adam (state0 = m, state1 = v, both [rows, C] fp32).
template <int NV>      // C = NV * 256
__global__ void table_update_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ order,
                                    const __nv_bfloat16* __restrict__ stage_g, const int* __restrict__ cnt_ptr, int cap,
                                    __nv_bfloat16* __restrict__ table, float* __restrict__ state0, float* __restrict__ state1, int mode, float lr,
                                    float beta1, float beta2, float eps, float decay, float c1, float c2, float inv_world, uint32_t seed,
                                    int* __restrict__ stats, long long rows_per_shard) {
  constexpr int C = NV * 256;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int n = min(*cnt_ptr, cap);
  if (i >= n) return;
  const long long id = sorted_ids[i];
  if (i > 0 && sorted_ids[i - 1] == id) return;           // not the head of its run
  if (!BONES_INDEX_OK(id, 0, rows_per_shard)) return;
  float acc[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[v][t] = 0.f;
  for (int j = i; j < n && sorted_ids[j] == id; ++j) {
    if (!BONES_INDEX_OK(order[j], 0, cap)) break;
    const __nv_bfloat16* src = stage_g + order[j] * (long long)C + lane * 8;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + v * 256);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float2 f = unpack_bf16(w[t]);
        acc[v][2 * t] += f.x;
        acc[v][2 * t + 1] += f.y;
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      acc[v][t] *= inv_world;
      ss += acc[v][t] * acc[v][t];
    }
  ss = warp_sum(ss);
  if (!isfinite(ss)) {
    if (lane == 0) atomicAdd(stats + 1, 1);
    return;
  }
  if (lane == 0) atomicAdd(stats, 1);
  __nv_bfloat16* w = table + id * (long long)C + lane * 8;
  float step_scale = 0.f;
  if (mode == 0) {
    float a = state0[id];
    a = beta2 * a + (1.0f - beta2) * ss / (float)C;
    __syncwarp();
    if (lane == 0) state0[id] = a;
    step_scale = lr / (sqrtf(a) + eps);
  }
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    uint4 u = *reinterpret_cast<const uint4*>(w + v * 256);
    uint32_t wd[4] = {u.x, u.y, u.z, u.w};
    float upd[8];
    if (mode == 0) {
#pragma unroll
      for (int t = 0; t < 8; ++t) upd[t] = step_scale * acc[v][t];
    } else {
      float* m = state0 + id * (long long)C + lane * 8 + v * 256;
      float* s = state1 + id * (long long)C + lane * 8 + v * 256;
      float4 m0 = *reinterpret_cast<float4*>(m), m1 = *reinterpret_cast<float4*>(m + 4);
      float4 s0 = *reinterpret_cast<float4*>(s), s1 = *reinterpret_cast<float4*>(s + 4);
      float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w}, sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        mm[t] += (1.0f - beta1) * (acc[v][t] - mm[t]);
        sv[t] += (1.0f - beta2) * (acc[v][t] * acc[v][t] - sv[t]);
        upd[t] = lr * (mm[t] / c1) / (sqrtf(sv[t] / c2) + eps);
      }
      *reinterpret_cast<float4*>(m) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(m + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
      *reinterpret_cast<float4*>(s) = make_float4(sv[0], sv[1], sv[2], sv[3]);
      *reinterpret_cast<float4*>(s + 4) = make_float4(sv[4], sv[5], sv[6], sv[7]);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 f = unpack_bf16(wd[t]);
      const float x0 = f.x * (1.0f - lr * decay) - upd[2 * t], x1 = f.y * (1.0f - lr * decay) - upd[2 * t + 1];
      // stochastic rounding to bf16: add 16 random bits below the kept mantissa, truncate
      const uint32_t rnd = tab_hash((uint32_t)id, (uint32_t)(lane * 8 + v * 256 + 2 * t), seed);
      const uint32_t b0 = (__float_as_uint(x0) + (rnd & 0xffffu)) >> 16, b1 = (__float_as_uint(x1) + (rnd >> 16)) >> 16;
      wd[t] = (isfinite(x0) ? b0 : (__float_as_uint(x0) >> 16)) | ((isfinite(x1) ? b1 : (__float_as_uint(x1) >> 16)) << 16);
    }
    *reinterpret_cast<uint4*>(w + v * 256) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
  }
}

__global__ void table_reset_kernel(long long* __restrict__ stage_ids, int* __restrict__ cnt, int cap) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = min(*cnt, cap);
  if (i < n) stage_ids[i] = kEmptyKey;
}
__global__ void table_zero_cnt_kernel(int* cnt) { *cnt = 0; }

static TabPeers tab_ptrs(void* const* ptrs, int world) {
  TabPeers p;
  for (int i = 0; i < kTabMaxPeers; ++i) p.p[i] = i < world ? ptrs[i] : nullptr;
  return p;
}

}  // namespace bones

extern "C" {
using namespace bones;

// ids [n] global row ids, g [n, C] bf16 gradient rows.  stage_*_ptrs: the W ranks' staging buffers (ids int64 [cap],
// rows bf16 [cap, C], counter int32 [1]).  overflow: local int32 counter of entries that found the owner's buffer full.
int bones_table_push(const long long* ids, const void* g, long long n, int C, void* const* stage_ids_ptrs, void* const* stage_g_ptrs,
                     void* const* stage_cnt_ptrs, int cap, int world, int* overflow, long long rows_per_shard, void* stream) {
  if (world > kTabMaxPeers || (C % 8)) return -2;
  if (n == 0) return 0;
  table_push_kernel<<<(unsigned)((n + 7) / 8), 256, 0, (cudaStream_t)stream>>>(ids, (const __nv_bfloat16*)g, n, C, tab_ptrs(stage_ids_ptrs, world),
                                                                              tab_ptrs(stage_g_ptrs, world), tab_ptrs(stage_cnt_ptrs, world), cap,
                                                                              world, overflow, rows_per_shard);
  return (int)cudaGetLastError();
}

// sorted_ids / order: the staged local ids sorted ascending (unused slots hold the empty key and sort last) and the
// permutation that sorted them.  stats[0] += rows updated, stats[1] += rows skipped for a non-finite gradient.
int bones_table_update(const long long* sorted_ids, const long long* order, const void* stage_g, const int* cnt, int cap, void* table, float* state0,
                       float* state1, int mode, int C, float lr, float beta1, float beta2, float eps, float decay, int step, float inv_world,
                       unsigned seed, int* stats, long long rows_per_shard, void* stream) {
  if ((C % 256) || C > 2048 || cap <= 0) return -2;
  const float c1 = 1.0f - powf(beta1, (float)step), c2 = 1.0f - powf(beta2, (float)step);
  const dim3 grid((unsigned)((cap + 7) / 8)), block(256);
  cudaStream_t st = (cudaStream_t)stream;
#define BONES_TAB_CASE(NV)                                                                                                                 \
  case NV:                                                                                                                                 \
    table_update_kernel<NV><<<grid, block, 0, st>>>(sorted_ids, order, (const __nv_bfloat16*)stage_g, cnt, cap, (__nv_bfloat16*)table, state0, \
                                                    state1, mode, lr, beta1, beta2, eps, decay, c1, c2, inv_world, seed, stats,           \
                                                    rows_per_shard);                                                                       \
    break;
  switch (C / 256) {
    BONES_TAB_CASE(1) BONES_TAB_CASE(2) BONES_TAB_CASE(3) BONES_TAB_CASE(4) BONES_TAB_CASE(5) BONES_TAB_CASE(6) BONES_TAB_CASE(7) BONES_TAB_CASE(8)
    default: return -2;
  }
#undef BONES_TAB_CASE
  return (int)cudaGetLastError();
}

int bones_table_reset(long long* stage_ids, int* cnt, int cap, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  table_reset_kernel<<<(unsigned)((cap + 255) / 256), 256, 0, st>>>(stage_ids, cnt, cap);
  table_zero_cnt_kernel<<<1, 1, 0, st>>>(cnt);
  return (int)cudaGetLastError();
}
}  // extern "C"
BONES_BOUNDS_EXPORT(tables)
