// Flash attention backward as two tcgen05 kernels (head_dim 128), the default backward of attention.cu's forward.
//
//   dkv kernel   one CTA per 128-key tile walks the query tiles that see it:  S = Qh Kh^T, dP = dO V^T,
//                P = exp2(S c1 - lse2) masked, dV += P^T dO, dS = P (dP - delta) scale, dK += dS^T Qh.
//   dq kernel    one CTA per 128-query tile walks its key tiles:  S and dP again, dS, dQ += dS Kh.
// Recomputing S and dP in the second kernel costs two extra GEMMs per tile pair, but every accumulator (dK, dV, dQ) then
// lives in TMEM for the whole CTA: no atomics, no per-tile drain, and the MMAs of the next tile pair are issued while
// the compute warps still work on the current one (in the single-kernel form, attention_bwd.cu, TMEM is full and the
// five GEMMs serialise with the exponentiation and a dQ drain through fp32 atomics).
// Operand views, masking, scaling and the saved statistics are those of attention_bwd.cu.
#include "common.cuh"

namespace bones {

constexpr int ST = 128;
constexpr uint32_t STILE = ST * 128 * 2;   // 32 KB: two 128-byte-swizzled atoms of [128 rows][64 cols]
constexpr uint32_t SATOM = STILE / 2;

struct SplitParams {
  int B, T, H;
  float c1, scale;
  int window_tiles;
  const int* doc_start;
  const float* lse;
  const float* delta;
  float* dqk;          // [B*T, 2A] fp32: dq-hat | dk-hat
  __nv_bfloat16* dv;   // [B*T, A]
  int* err;
};

__device__ __forceinline__ int split_first_tile(const SplitParams& p, int b, int qt) {
  int lo = 0;
  if (p.doc_start) lo = p.doc_start[(long long)b * p.T + qt * ST] / ST;
  if (p.window_tiles > 0) lo = max(lo, qt - p.window_tiles + 1);
  return lo;
}
__device__ __forceinline__ uint64_t sdesc_k(uint32_t tile, int k) {   // K-major view, UMMA_K step k
  return umma_smem_desc(tile + (k >> 2) * SATOM + (k & 3) * 32, 0, 1024, kLayoutSw128);
}
__device__ __forceinline__ uint64_t sdesc_mn(uint32_t tile, int k) {  // MN-major view of the same bytes
  return umma_smem_desc(tile + k * 2048, SATOM, 1024, kLayoutSw128);
}
__device__ __forceinline__ void store_row64_sw128(uint32_t tile, int half, int r, const float* v) {
  const uint32_t prow = tile + (uint32_t)half * SATOM + (uint32_t)r * 128u;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const uint32_t chunk = (uint32_t)g ^ (uint32_t)(r & 7);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + chunk * 16u), "r"(pack_bf16(v[g * 8 + 0], v[g * 8 + 1])),
                 "r"(pack_bf16(v[g * 8 + 2], v[g * 8 + 3])), "r"(pack_bf16(v[g * 8 + 4], v[g * 8 + 5])),
                 "r"(pack_bf16(v[g * 8 + 6], v[g * 8 + 7]))
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// dK / dV
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(320, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_qk, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_dy, const SplitParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sK = base, sV = base + STILE;
  auto sQ = [&](int s) { return base + STILE * (2 + 2 * s); };
  auto sdO = [&](int s) { return base + STILE * (3 + 2 * s); };
  const uint32_t sPB = base + STILE * 6;
  const uint32_t bars = base + STILE * 7;
  enum { B_KV = 0, B_QDO0, B_QDO1, B_FREE0, B_FREE1, B_SFULL, B_DPFULL, B_PREADY, B_DVDONE, B_DSREADY, B_DKDONE, B_COUNT };
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t tmem_slot = bars + 8u * B_COUNT;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + STILE * 7 + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + STILE * 7 + 8 * B_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int A = p.H * 128;
  const int n_tiles = p.T / ST;

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
    mbar_init(bar(B_DKDONE), 1);
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

  int n = 0;
  for (int qt = kt; qt < n_tiles; ++qt) {
    if (split_first_tile(p, b, qt) > kt) break;
    ++n;
  }
  const int row0 = b * p.T;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(B_KV), 2 * STILE);
      tma_load_2d(sK, &tm_qk, bar(B_KV), A + h * 128, row0 + kt * ST);
      tma_load_2d(sK + SATOM, &tm_qk, bar(B_KV), A + h * 128 + 64, row0 + kt * ST);
      tma_load_2d(sV, &tm_v, bar(B_KV), 2 * A + h * 128, row0 + kt * ST);
      tma_load_2d(sV + SATOM, &tm_v, bar(B_KV), 2 * A + h * 128 + 64, row0 + kt * ST);
      for (int i = 0; i < n; ++i) {
        const int s = i & 1;
        if (i >= 2 && !mbar_wait(bar(B_FREE0 + s), ((i - 2) >> 1) & 1, abort_flag, p.err, ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(bar(B_QDO0 + s), 2 * STILE);
        const int r = row0 + (kt + i) * ST;
        tma_load_2d(sQ(s), &tm_qk, bar(B_QDO0 + s), h * 128, r);
        tma_load_2d(sQ(s) + SATOM, &tm_qk, bar(B_QDO0 + s), h * 128 + 64, r);
        tma_load_2d(sdO(s), &tm_dy, bar(B_QDO0 + s), h * 128, r);
        tma_load_2d(sdO(s) + SATOM, &tm_dy, bar(B_QDO0 + s), h * 128 + 64, r);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = umma_idesc_f16(128, 128, 1, 0, 0);
      const uint32_t id_mm = umma_idesc_f16(128, 128, 1, 1, 1);
      bool ok = mbar_wait(bar(B_KV), 0, abort_flag, p.err, ERR_WAIT_FULL);
      // S(0), dP(0)
      if (ok && n > 0) {
        ok = mbar_wait(bar(B_QDO0), 0, abort_flag, p.err, ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tS, sdesc_k(sQ(0), k), sdesc_k(sK, k), id_kk, k ? 1u : 0u);
          tc_commit(bar(B_SFULL));
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tdP, sdesc_k(sdO(0), k), sdesc_k(sV, k), id_kk, k ? 1u : 0u);
          tc_commit(bar(B_DPFULL));
        }
      }
      for (int i = 0; i < n && ok; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i & 1);
        const bool more = i + 1 < n;
        // P(i) is in shared memory (and S(i) has been read): dV += P^T dO, then S(i+1) behind it
        if (!mbar_wait(bar(B_PREADY), ph, abort_flag, p.err, ERR_WAIT_AUX)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdV, sdesc_mn(sPB, k), sdesc_mn(sdO(s), k), id_mm, (i | k) ? 1u : 0u);
        tc_commit(bar(B_DVDONE));
        if (more) {
          if (!mbar_wait(bar(B_QDO0 + (s ^ 1)), ((i + 1) >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tS, sdesc_k(sQ(s ^ 1), k), sdesc_k(sK, k), id_kk, k ? 1u : 0u);
          tc_commit(bar(B_SFULL));
        }
        // dS(i) is in shared memory (and dP(i) has been read): dK += dS^T Qh, then dP(i+1) behind it
        if (!mbar_wait(bar(B_DSREADY), ph, abort_flag, p.err, ERR_WAIT_AUX)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdK, sdesc_mn(sPB, k), sdesc_mn(sQ(s), k), id_mm, (i | k) ? 1u : 0u);
        tc_commit(bar(B_DKDONE));
        tc_commit(bar(B_FREE0 + s));
        if (more) {
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tdP, sdesc_k(sdO(s ^ 1), k), sdesc_k(sV, k), id_kk, k ? 1u : 0u);
          tc_commit(bar(B_DPFULL));
        }
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int c0 = half * 64;
    const float log2e = 1.4426950408889634f;
    bool ok = true;
    float nx_lse2 = 0.f, nx_dlt = 0.f;
    int nx_lo = 0;
    if (n > 0) {
      const int qpos0 = kt * ST + r;
      const long long st0 = ((long long)b * p.H + h) * p.T + qpos0;
      nx_lse2 = p.lse[st0] * log2e;
      nx_dlt = p.delta[st0];
      if (p.doc_start) nx_lo = p.doc_start[(long long)b * p.T + qpos0];
    }
    for (int i = 0; i < n && ok; ++i) {
      const uint32_t ph = (uint32_t)(i & 1);
      const int qpos = (kt + i) * ST + r;
      const float lse2 = nx_lse2, dlt = nx_dlt;
      const int lo = nx_lo;
      if (i + 1 < n) {
        const int qn = qpos + ST;
        const long long stn = ((long long)b * p.H + h) * p.T + qn;
        nx_lse2 = p.lse[stn] * log2e;
        nx_dlt = p.delta[stn];
        if (p.doc_start) nx_lo = p.doc_start[(long long)b * p.T + qn];
      }
      const int k0 = kt * ST;
      const bool need_mask = __any_sync(0xffffffffu, (i == 0) || (k0 + c0 < lo));
      float pr[64];
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
          const float xx = fmaf(__uint_as_float(v[j]), p.c1, -lse2);
          float e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(xx));
          pr[c * 32 + j] = e;
        }
      }
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int kpos = k0 + c0 + j;
          if (kpos > qpos || kpos < lo) pr[j] = 0.f;
        }
      }
      tc_fence_before();
      if (i >= 1) {   // dS(i-1) must have been consumed by dK's MMAs before P(i) overwrites the buffer
        got = mbar_wait(bar(B_DKDONE), (uint32_t)((i - 1) & 1), abort_flag, p.err, ERR_WAIT_AUX);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      }
      store_row64_sw128(sPB, half, r, pr);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PREADY));
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
      got = mbar_wait(bar(B_DVDONE), ph, abort_flag, p.err, ERR_WAIT_AUX);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      store_row64_sw128(sPB, half, r, pr);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DSREADY));
    }
    if (ok && n > 0) {
      const bool got = mbar_wait(bar(B_DKDONE), (uint32_t)((n - 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        const int kpos = kt * ST + r;
        float* dk = p.dqk + ((long long)(row0 + kpos)) * 2 * A + A + (long long)h * 128 + c0;
        __nv_bfloat16* dv = p.dv + ((long long)(row0 + kpos)) * A + (long long)h * 128 + c0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          __syncwarp();
          BONES_TMEM_LD32(tdK + lane_addr + (uint32_t)(c0 + c * 32), v);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(dk + c * 32 + g * 4) = make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]),
                                                                          __uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3]));
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

// ---------------------------------------------------------------------------------------------------------------
// dQ
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qk, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_dy, const SplitParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sQ = base, sdO = base + STILE;
  auto sK = [&](int s) { return base + STILE * (2 + 2 * s); };
  auto sV = [&](int s) { return base + STILE * (3 + 2 * s); };
  const uint32_t sDS = base + STILE * 6;
  const uint32_t bars = base + STILE * 7;
  enum { B_QDO = 0, B_KV0, B_KV1, B_FREE0, B_FREE1, B_SDP0, B_SDP1, B_DSREADY, B_DQDONE, B_COUNT };
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t tmem_slot = bars + 8u * B_COUNT;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + STILE * 7 + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + STILE * 7 + 8 * B_COUNT + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int A = p.H * 128;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QDO), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(B_KV0 + s), 1);
      mbar_init(bar(B_FREE0 + s), 1);
      mbar_init(bar(B_SDP0 + s), 1);
    }
    mbar_init(bar(B_DSREADY), 8);
    mbar_init(bar(B_DQDONE), 1);
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
  // S and dP are double-buffered as pairs: buffer s holds S at +0 and dP at +128 of its 256 columns?  No: dQ needs 128
  // columns too, so S is double-buffered (0, 128), dP single (256), dQ (384).
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tdP = tmem + 256, tdQ = tmem + 384;

  const int kt0 = split_first_tile(p, b, qt);
  const int n = qt - kt0 + 1;
  const int row0 = b * p.T;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(B_QDO), 2 * STILE);
      const int rq = row0 + qt * ST;
      tma_load_2d(sQ, &tm_qk, bar(B_QDO), h * 128, rq);
      tma_load_2d(sQ + SATOM, &tm_qk, bar(B_QDO), h * 128 + 64, rq);
      tma_load_2d(sdO, &tm_dy, bar(B_QDO), h * 128, rq);
      tma_load_2d(sdO + SATOM, &tm_dy, bar(B_QDO), h * 128 + 64, rq);
      for (int j = 0; j < n; ++j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(bar(B_FREE0 + s), ((j - 2) >> 1) & 1, abort_flag, p.err, ERR_WAIT_EMPTY)) break;
        mbar_arrive_expect_tx(bar(B_KV0 + s), 2 * STILE);
        const int r = row0 + (kt0 + j) * ST;
        tma_load_2d(sK(s), &tm_qk, bar(B_KV0 + s), A + h * 128, r);
        tma_load_2d(sK(s) + SATOM, &tm_qk, bar(B_KV0 + s), A + h * 128 + 64, r);
        tma_load_2d(sV(s), &tm_v, bar(B_KV0 + s), 2 * A + h * 128, r);
        tma_load_2d(sV(s) + SATOM, &tm_v, bar(B_KV0 + s), 2 * A + h * 128 + 64, r);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_kk = umma_idesc_f16(128, 128, 1, 0, 0);
      const uint32_t id_km = umma_idesc_f16(128, 128, 1, 0, 1);
      bool ok = mbar_wait(bar(B_QDO), 0, abort_flag, p.err, ERR_WAIT_FULL);
      for (int j = 0; j < n && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(B_KV0 + s), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        // S(j): its buffer was last read for tile j-2, whose dS has long been published
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tS[s], sdesc_k(sQ, k), sdesc_k(sK(s), k), id_kk, k ? 1u : 0u);
        if (j >= 1) {
          // dS(j-1) is in shared memory and dP(j-1) has been read: dQ += dS Kh(j-1), which also frees that K/V stage
          if (!mbar_wait(bar(B_DSREADY), (uint32_t)((j - 1) & 1), abort_flag, p.err, ERR_WAIT_AUX)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tdQ, sdesc_k(sDS, k), sdesc_mn(sK(s ^ 1), k), id_km, ((j - 1) | k) ? 1u : 0u);
          tc_commit(bar(B_DQDONE));
          tc_commit(bar(B_FREE0 + (s ^ 1)));
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdP, sdesc_k(sdO, k), sdesc_k(sV(s), k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_SDP0 + s));
      }
      if (ok && n > 0) {
        const int s = (n - 1) & 1;
        if (mbar_wait(bar(B_DSREADY), (uint32_t)((n - 1) & 1), abort_flag, p.err, ERR_WAIT_AUX)) {
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16(tdQ, sdesc_k(sDS, k), sdesc_mn(sK(s), k), id_km, ((n - 1) | k) ? 1u : 0u);
          tc_commit(bar(B_DQDONE));
        }
      }
    }
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int c0 = half * 64;
    const int qpos = qt * ST + r;
    const long long stat = ((long long)b * p.H + h) * p.T + qpos;
    const float lse2 = p.lse[stat] * 1.4426950408889634f;
    const float dlt = p.delta[stat];
    int lo = 0;
    if (p.doc_start) lo = p.doc_start[(long long)b * p.T + qpos];
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      const int s = j & 1;
      bool got = mbar_wait(bar(B_SDP0 + s), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      const int k0 = (kt0 + j) * ST + c0;
      const bool need_mask = __any_sync(0xffffffffu, (k0 + 63 > qpos) || (k0 < lo));
      float pr[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32], w[32];
        __syncwarp();
        BONES_TMEM_LD32(tS[s] + lane_addr + (uint32_t)(c0 + c * 32), v);
        BONES_TMEM_LD32(tdP + lane_addr + (uint32_t)(c0 + c * 32), w);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float xx = fmaf(__uint_as_float(v[i]), p.c1, -lse2);
          float e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(xx));
          pr[c * 32 + i] = e * (__uint_as_float(w[i]) - dlt) * p.scale;
        }
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int kpos = k0 + i;
          if (kpos > qpos || kpos < lo) pr[i] = 0.f;
        }
      }
      tc_fence_before();
      if (j >= 1) {   // the dQ MMAs of tile j-1 must be done reading the dS buffer
        got = mbar_wait(bar(B_DQDONE), (uint32_t)((j - 1) & 1), abort_flag, p.err, ERR_WAIT_AUX);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      }
      store_row64_sw128(sDS, half, r, pr);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DSREADY));
    }
    if (ok && n > 0) {
      const bool got = mbar_wait(bar(B_DQDONE), (uint32_t)((n - 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        float* dq = p.dqk + ((long long)(row0 + qpos)) * 2 * A + (long long)h * 128 + c0;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          __syncwarp();
          BONES_TMEM_LD32(tdQ + lane_addr + (uint32_t)(c0 + c * 32), v);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(dq + c * 32 + g * 4) = make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]),
                                                                          __uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3]));
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

static int tmap_rows_2d_s(CUtensorMap* out, const void* ptr, long long rows, long long cols) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  uint64_t strides[1] = {(uint64_t)cols * 2};
  uint32_t box[2] = {64, 128};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace bones

extern "C" {
using namespace bones;

// Same contract as bones_attn_bwd (attention_bwd.cu); dqk needs no zeroing: both halves are overwritten.
int bones_attn_bwd_split(const void* qk, const void* qkv, const void* dy, const float* lse, const float* delta, float* dqk, void* dv,
                         const int* doc_start, int B, int T, int H, float scale, int window_tiles, void* stream) {
  if (T % ST) return -2;
  const long long M = (long long)B * T, A = (long long)H * 128;
  CUtensorMap tq, tv, td;
  int rc = tmap_rows_2d_s(&tq, qk, M, 2 * A);
  if (rc) return rc;
  rc = tmap_rows_2d_s(&tv, qkv, M, 3 * A);
  if (rc) return rc;
  rc = tmap_rows_2d_s(&td, dy, M, A);
  if (rc) return rc;
  SplitParams p;
  p.B = B; p.T = T; p.H = H;
  p.c1 = scale * 1.4426950408889634f;
  p.scale = scale;
  p.window_tiles = window_tiles;
  p.doc_start = doc_start;
  p.lse = lse; p.delta = delta; p.dqk = dqk; p.dv = (__nv_bfloat16*)dv;
  p.err = error_word();
  constexpr size_t smem = (size_t)STILE * 7 + 160 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    BONES_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  dim3 grid(T / ST, H, B);
  cudaStream_t s = (cudaStream_t)stream;
  attn_bwd_dkv_kernel<<<grid, 320, smem, s>>>(tq, tv, td, p);
  BONES_CHECK(cudaGetLastError());
  attn_bwd_dq_kernel<<<grid, 320, smem, s>>>(tq, tv, td, p);
  return (int)cudaGetLastError();
}
}  // extern "C"
