// Causal flash attention backward on tcgen05 tensor cores (head_dim 128), for the forward in attention.cu.
//
// One CTA per (128-key tile, head, batch) walks the query tiles that can see it.  Per query tile (reference math:
// `P = exp(scale*S - lse)`, `dS = P * (dP - D)`, round2/source/kernels/nki_attn_bandpro.py:1-134):
//     S  = Qh Kh^T            dP = dO V^T                      (tensor core -> TMEM)
//     P  = exp2(S*c1 - lse2)  masked                           (one half-row per thread, written bf16 to shared memory)
//     dV += P^T dO                                             (accumulates in TMEM over the query tiles)
//     dS = P * (dP - delta) * scale                            (overwrites P in shared memory once dV's MMAs are done)
//     dK += dS^T Qh           dQ = dS Kh                       (dK accumulates in TMEM; dQ is drained per tile)
// dQ tiles are added to an fp32 buffer with vector atomics (several key tiles contribute to one query tile); dK/dV leave
// the CTA once, at the end.  The same shared-memory tile serves as a K-major or an MN-major operand just by changing the
// UMMA descriptor, so no transposed copies exist: P^T, dS^T, dO^T and Kh^T are descriptor views.
//
// Warp roles: warp 0 TMA producer (Kh, V once; Qh, dO double-buffered), warp 1 MMA issuer + TMEM owner, warps 2-9
// compute (two warps per 32-lane TMEM quadrant, 64 columns each).  TMEM: S/dQ | dP | dV | dK = 4 x 128 columns.
#include <mutex>

#include "bones_noalloc.h"
#include "common.cuh"

namespace bones {

constexpr int BT = 128;
constexpr int BD = 128;
constexpr uint32_t BTILE = BT * BD * 2;    // 32 KB
constexpr uint32_t BATOM = BTILE / 2;

struct AttnBwdParams {
  int B, T, H;
  float c1;            // scale * log2(e)
  float scale;
  int window_tiles;
  const int* doc_start;
  const float* lse;    // [B, H, T]
  const float* delta;  // [B, H, T]
  float* dqk;          // [B*T, 2*A] fp32: dq-hat (atomically accumulated) | dk-hat
  __nv_bfloat16* dv;   // [B*T, A]
  int* err;
};

__device__ __forceinline__ int bwd_first_tile(const AttnBwdParams& p, int b, int qt) {
  int lo = 0;
  if (p.doc_start) lo = p.doc_start[(long long)b * p.T + qt * BT] / BT;
  if (p.window_tiles > 0) lo = max(lo, qt - p.window_tiles + 1);
  return lo;
}

// delta[b,h,t] = sum_d dO * O
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y, float* __restrict__ delta,
                                  long long M, int T, int H) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= M * H) return;
  const int h = (int)(w % H);
  const long long row = w / H;
  const long long off = row * H * BD + (long long)h * BD + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(dy + off), c = *reinterpret_cast<const uint2*>(y + off);
  const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), c0 = unpack_bf16(c.x), c1 = unpack_bf16(c.y);
  float s = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y;
  s = warp_sum(s);
  if (lane == 0) {
    const long long b = row / T, t = row % T;
    delta[(b * H + h) * T + t] = s;
  }
}

__global__ void __launch_bounds__(320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qk, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_dy, const AttnBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sK = base, sV = base + BTILE;
  auto sQ = [&](int s) { return base + BTILE * (2 + 2 * s); };
  auto sdO = [&](int s) { return base + BTILE * (3 + 2 * s); };
  const uint32_t sPB = base + BTILE * 6;
  const uint32_t bars = base + BTILE * 7;
  enum { B_KV = 0, B_QDO0, B_QDO1, B_FREE0, B_FREE1, B_SFULL, B_DPFULL, B_PREADY, B_DVDONE, B_DSREADY, B_DQFULL, B_DQREAD, B_COUNT };
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t tmem_slot = bars + 8u * B_COUNT;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + BTILE * 7 + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + BTILE * 7 + 8 * B_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int A = p.H * BD;
  const int n_tiles = p.T / BT;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_KV), 1);
    mbar_init(bar(B_QDO0), 1);
    mbar_init(bar(B_QDO1), 1);
    mbar_init(bar(B_FREE0), 1);
    mbar_init(bar(B_FREE1), 1);
    mbar_init(bar(B_SFULL), 1);
    mbar_init(bar(B_DPFULL), 1);
    mbar_init(bar(B_PREADY), 8);
    mbar_init(bar(B_DVDONE), 1);
    mbar_init(bar(B_DSREADY), 8);
    mbar_init(bar(B_DQFULL), 1);
    mbar_init(bar(B_DQREAD), 8);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_qk);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_dy);
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
  const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

  // query tiles that see this key tile: kt, kt+1, ... while the tile's first visible key tile is <= kt
  int n = 0;
  for (int qt = kt; qt < n_tiles; ++qt) {
    if (bwd_first_tile(p, b, qt) > kt) break;
    ++n;
  }
  const int row0 = b * p.T;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(B_KV), 2 * BTILE);
      tma_load_2d(sK, &tm_qk, bar(B_KV), A + h * BD, row0 + kt * BT);
      tma_load_2d(sK + BATOM, &tm_qk, bar(B_KV), A + h * BD + 64, row0 + kt * BT);
      tma_load_2d(sV, &tm_v, bar(B_KV), 2 * A + h * BD, row0 + kt * BT);
      tma_load_2d(sV + BATOM, &tm_v, bar(B_KV), 2 * A + h * BD + 64, row0 + kt * BT);
      for (int i = 0; i < n; ++i) {
        const int s = i & 1;
        if (i >= 2 && !mbar_wait(bar(B_FREE0 + s), ((i - 2) >> 1) & 1, abort_flag, p.err, ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(bar(B_QDO0 + s), 2 * BTILE);
        const int r = row0 + (kt + i) * BT;
        tma_load_2d(sQ(s), &tm_qk, bar(B_QDO0 + s), h * BD, r);
        tma_load_2d(sQ(s) + BATOM, &tm_qk, bar(B_QDO0 + s), h * BD + 64, r);
        tma_load_2d(sdO(s), &tm_dy, bar(B_QDO0 + s), h * BD, r);
        tma_load_2d(sdO(s) + BATOM, &tm_dy, bar(B_QDO0 + s), h * BD + 64, r);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = umma_idesc_f16(128, 128, 1, 0, 0);   // both K-major
      const uint32_t id_mm = umma_idesc_f16(128, 128, 1, 1, 1);   // both MN-major
      const uint32_t id_km = umma_idesc_f16(128, 128, 1, 0, 1);   // A K-major, B MN-major
      auto kmaj = [&](uint32_t tile, int k) { return umma_smem_desc(tile + (k >> 2) * BATOM + (k & 3) * 32, 0, 1024, kLayoutSw128); };
      auto mnmaj = [&](uint32_t tile, int k) { return umma_smem_desc(tile + k * 2048, BATOM, 1024, kLayoutSw128); };
      bool ok = mbar_wait(bar(B_KV), 0, abort_flag, p.err, ERR_WAIT_FULL);
      for (int i = 0; i < n && ok; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i & 1);
        if (!mbar_wait(bar(B_QDO0 + s), (i >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        // dP = dO V^T (tdP is free: the previous tile's dP was consumed before its dS was published)
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdP, kmaj(sdO(s), k), kmaj(sV, k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_DPFULL));
        // S = Qh Kh^T needs tS back from the previous tile's dQ drain
        if (i >= 1 && !mbar_wait(bar(B_DQREAD), (uint32_t)((i - 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tS, kmaj(sQ(s), k), kmaj(sK, k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_SFULL));
        // dV += P^T dO
        if (!mbar_wait(bar(B_PREADY), ph, abort_flag, p.err, ERR_WAIT_AUX)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdV, mnmaj(sPB, k), mnmaj(sdO(s), k), id_mm, (i | k) ? 1u : 0u);
        tc_commit(bar(B_DVDONE));
        // dK += dS^T Qh ; dQ = dS Kh
        if (!mbar_wait(bar(B_DSREADY), ph, abort_flag, p.err, ERR_WAIT_AUX)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdK, mnmaj(sPB, k), mnmaj(sQ(s), k), id_mm, (i | k) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tS, kmaj(sPB, k), mnmaj(sK, k), id_km, k ? 1u : 0u);
        tc_commit(bar(B_DQFULL));
        tc_commit(bar(B_FREE0 + s));
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int c0 = half * 64;
    const float log2e = 1.4426950408889634f;
    bool ok = true;
    // per-row statistics of the next query tile are fetched one iteration ahead so their latency hides behind the MMAs
    float nx_lse2 = 0.f, nx_dlt = 0.f;
    int nx_lo = 0;
    if (n > 0) {
      const int qpos0 = kt * BT + r;
      const long long st0 = ((long long)b * p.H + h) * p.T + qpos0;
      nx_lse2 = p.lse[st0] * log2e;
      nx_dlt = p.delta[st0];
      if (p.doc_start) nx_lo = p.doc_start[(long long)b * p.T + qpos0];
    }
    for (int i = 0; i < n && ok; ++i) {
      const uint32_t ph = (uint32_t)(i & 1);
      const int qt = kt + i;
      const int qpos = qt * BT + r;
      const float lse2 = nx_lse2, dlt = nx_dlt;
      const int lo = nx_lo;
      if (i + 1 < n) {
        const int qn = qpos + BT;
        const long long stn = ((long long)b * p.H + h) * p.T + qn;
        nx_lse2 = p.lse[stn] * log2e;
        nx_dlt = p.delta[stn];
        if (p.doc_start) nx_lo = p.doc_start[(long long)b * p.T + qn];
      }
      const int k0 = kt * BT;
      const bool need_mask = __any_sync(0xffffffffu, (i == 0) || (k0 + c0 < lo));
      float pr[64];
      // ---- P ----
      bool got = mbar_wait(bar(B_SFULL), ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        __syncwarp();
        BONES_TMEM_LD32(tS + lane_addr + (uint32_t)(c0 + c * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float e;
          const float xx = fmaf(__uint_as_float(v[j]), p.c1, -lse2);
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(xx));
          if (need_mask) {
            const int kpos = k0 + c0 + c * 32 + j;
            if (kpos > qpos || kpos < lo) e = 0.f;
          }
          pr[c * 32 + j] = e;
        }
      }
      const uint32_t prow = sPB + (uint32_t)half * BATOM + (uint32_t)r * 128u;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const uint32_t chunk = (uint32_t)g ^ (uint32_t)(r & 7);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + chunk * 16u), "r"(pack_bf16(pr[g * 8 + 0], pr[g * 8 + 1])),
                     "r"(pack_bf16(pr[g * 8 + 2], pr[g * 8 + 3])), "r"(pack_bf16(pr[g * 8 + 4], pr[g * 8 + 5])),
                     "r"(pack_bf16(pr[g * 8 + 6], pr[g * 8 + 7]))
                     : "memory");
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PREADY));
      // ---- dS ----
      got = mbar_wait(bar(B_DPFULL), ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        __syncwarp();
        BONES_TMEM_LD32(tdP + lane_addr + (uint32_t)(c0 + c * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) pr[c * 32 + j] = pr[c * 32 + j] * (__uint_as_float(v[j]) - dlt) * p.scale;
      }
      tc_fence_before();
      got = mbar_wait(bar(B_DVDONE), ph, abort_flag, p.err, ERR_WAIT_AUX);    // P no longer being read by dV's MMAs
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const uint32_t chunk = (uint32_t)g ^ (uint32_t)(r & 7);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + chunk * 16u), "r"(pack_bf16(pr[g * 8 + 0], pr[g * 8 + 1])),
                     "r"(pack_bf16(pr[g * 8 + 2], pr[g * 8 + 3])), "r"(pack_bf16(pr[g * 8 + 4], pr[g * 8 + 5])),
                     "r"(pack_bf16(pr[g * 8 + 6], pr[g * 8 + 7]))
                     : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DSREADY));
      // ---- dQ drain ----
      got = mbar_wait(bar(B_DQFULL), ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      float* dq = p.dqk + ((long long)(row0 + qpos)) * 2 * A + (long long)h * BD + c0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        __syncwarp();
        BONES_TMEM_LD32(tS + lane_addr + (uint32_t)(c0 + c * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          atomicAdd(reinterpret_cast<float4*>(dq + c * 32 + g * 4),
                    make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]), __uint_as_float(v[g * 4 + 2]),
                                __uint_as_float(v[g * 4 + 3])));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DQREAD));
    }
    if (ok && n > 0) {
      // every MMA of the last tile was committed to B_DQFULL, which this thread has already observed
      const int kpos = kt * BT + r;
      float* dk = p.dqk + ((long long)(row0 + kpos)) * 2 * A + A + (long long)h * BD + c0;
      __nv_bfloat16* dv = p.dv + ((long long)(row0 + kpos)) * A + (long long)h * BD + c0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        __syncwarp();
        BONES_TMEM_LD32(tdK + lane_addr + (uint32_t)(c0 + c * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<float4*>(dk + c * 32 + g * 4) =
              make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]), __uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3]));
        __syncwarp();
        BONES_TMEM_LD32(tdV + lane_addr + (uint32_t)(c0 + c * 32), v);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 u;
          u.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
          u.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
          u.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
          u.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
          *reinterpret_cast<uint4*>(dv + c * 32 + g * 8) = u;
        }
      }
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

static int tmap_rows_2d_b(CUtensorMap* out, const void* ptr, long long rows, long long cols) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)cols * 2};
  uint32_t box[2] = {64, 128};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace bones

extern "C" {
using namespace bones;

int bones_attn_delta(const void* dy, const void* y, float* delta, long long M, int T, int H, void* stream) {
  const long long warps = M * H;
  attn_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, delta, M, T, H);
  return (int)cudaGetLastError();
}

// dqk: fp32 [B*T, 2A]; its dq half is zeroed here and accumulated atomically, its dk half is overwritten.  dv: bf16 [B*T, A].
int bones_attn_bwd(const void* qk, const void* qkv, const void* dy, const float* lse, const float* delta, float* dqk, void* dv,
                   const int* doc_start, int B, int T, int H, float scale, int window_tiles, void* stream) {
  if (T % BT) return -2;
  const long long M = (long long)B * T, A = (long long)H * BD;
  CUtensorMap tq, tv, td;
  int rc = tmap_rows_2d_b(&tq, qk, M, 2 * A);
  if (rc) return rc;
  rc = tmap_rows_2d_b(&tv, qkv, M, 3 * A);
  if (rc) return rc;
  rc = tmap_rows_2d_b(&td, dy, M, A);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  BONES_CHECK(cudaMemset2DAsync(dqk, (size_t)(2 * A) * 4, 0, (size_t)A * 4, (size_t)M, s));
  AttnBwdParams p;
  p.B = B; p.T = T; p.H = H;
  p.c1 = scale * 1.4426950408889634f;
  p.scale = scale;
  p.window_tiles = window_tiles;
  p.doc_start = doc_start;
  p.lse = lse; p.delta = delta; p.dqk = dqk; p.dv = (__nv_bfloat16*)dv;
  p.err = error_word();
  constexpr size_t smem = (size_t)BTILE * 7 + 160 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  dim3 grid(T / BT, H, B);
  attn_bwd_kernel<<<grid, 320, smem, s>>>(tq, tv, td, p);
  return (int)cudaGetLastError();
}
}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the attention backward (declared in bones_noalloc.h).
// ---------------------------------------------------------------------------------------------------------------
namespace bones {
// delta = rowsum(dO * O) is the one piece of scratch the backward needs besides its inputs and outputs.  It lives here, in
// a fixed array every GPU that loads this library keeps until the process exits (4 MiB), instead of coming from
// cudaMalloc or a framework allocator.
constexpr long long kNoAllocMaxRows = 1ll << 20;        // B * H * T
static __device__ __align__(256) float g_noalloc_delta[kNoAllocMaxRows];
static __device__ __align__(256) int g_noalloc_err[64];

struct NoAllocDevice {
  float* delta = nullptr;   // device addresses resolved from the symbols above (the symbol names are host stand-ins)
  int* err = nullptr;
  bool ready = false;       // symbol addresses resolved
  bool attr = false;        // the kernel's shared-memory limit has been raised
};
static NoAllocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_mu;      // guards the per-device set-up: two host threads may make the first call at once

// Resolves the scratch and error-word addresses of the current device once.  0 or a negative set-up code.
static int noalloc_setup(int dev, size_t smem, NoAllocDevice** out) {
  if (dev < 0 || dev >= 64) return -12;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  NoAllocDevice& nd = g_noalloc_dev[dev];
  if (!nd.ready) {
    // once per device, with that device current: turn the symbols into device addresses
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_delta) != cudaSuccess || !p) return -11;
    nd.delta = static_cast<float*>(p);
    if (cudaGetSymbolAddress(&p, g_noalloc_err) != cudaSuccess || !p) return -11;
    nd.err = static_cast<int*>(p);
    nd.ready = true;
  }
  if (smem && !nd.attr) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    nd.attr = true;
  }
  *out = &nd;
  return 0;
}
}  // namespace bones

extern "C" {
using namespace bones;

const char* bones_attn_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -2: return "sequence length must be a multiple of 128";
    case -10: return "B*H*T exceeds the built-in scratch (1048576 rows): split the batch or use bones_attn_bwd";
    case -11: return "could not resolve the scratch symbol on this device (cudaGetSymbolAddress failed)";
    case -12: return "unsupported device ordinal (>= 64)";
    default: return code > 0 ? "CUDA runtime error (the value is the cudaError_t)" : "tensor-map encoding failed";
  }
}

int bones_attn_bwd_noalloc(const void* qk, const void* qkv, const void* dy, const void* y, const float* lse, float* dqk, void* dv,
                           const int* doc_start, int B, int T, int H, float scale, int window_tiles, void* stream) {
  if (T % BT) return -2;
  const long long M = (long long)B * T, A = (long long)H * BD;
  if (M * H > kNoAllocMaxRows) return -10;
  int dev = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  constexpr size_t smem = (size_t)BTILE * 7 + 160 + 1024;
  NoAllocDevice* ndp = nullptr;
  const int src = noalloc_setup(dev, smem, &ndp);
  if (src) return src;
  NoAllocDevice& nd = *ndp;
  CUtensorMap tq, tv, td;
  int rc = tmap_rows_2d_b(&tq, qk, M, 2 * A);
  if (rc) return rc;
  rc = tmap_rows_2d_b(&tv, qkv, M, 3 * A);
  if (rc) return rc;
  rc = tmap_rows_2d_b(&td, dy, M, A);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const long long warps = M * H;
  attn_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y, nd.delta, M, T, H);
  BONES_CHECK(cudaGetLastError());
  BONES_CHECK(cudaMemset2DAsync(dqk, (size_t)(2 * A) * 4, 0, (size_t)A * 4, (size_t)M, s));
  AttnBwdParams p;
  p.B = B; p.T = T; p.H = H;
  p.c1 = scale * 1.4426950408889634f;
  p.scale = scale;
  p.window_tiles = window_tiles;
  p.doc_start = doc_start;
  p.lse = lse; p.delta = nd.delta; p.dqk = dqk; p.dv = (__nv_bfloat16*)dv;
  p.err = nd.err;
  dim3 grid(T / BT, H, B);
  attn_bwd_kernel<<<grid, 320, smem, s>>>(tq, tv, td, p);
  return (int)cudaGetLastError();
}

// Status of the calls made so far on the current device: 0, or the code of the first bounded wait that ran out inside
// the kernel since the last read (the call itself had returned 0: launches are asynchronous).  Waits for `stream`, copies
// one word out of the library's own error word and clears it; allocates nothing.
int bones_attn_bwd_noalloc_error_read_clear(void* stream) {
  int dev = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  NoAllocDevice* ndp = nullptr;
  const int src = noalloc_setup(dev, 0, &ndp);
  if (src) return src;
  cudaStream_t s = (cudaStream_t)stream;
  int v = 0;
  BONES_CHECK(cudaMemcpyAsync(&v, ndp->err, sizeof(int), cudaMemcpyDeviceToHost, s));
  BONES_CHECK(cudaStreamSynchronize(s));
  if (v != 0) {
    BONES_CHECK(cudaMemsetAsync(ndp->err, 0, sizeof(int), s));
    BONES_CHECK(cudaStreamSynchronize(s));
  }
  return v;
}
}  // extern "C"
