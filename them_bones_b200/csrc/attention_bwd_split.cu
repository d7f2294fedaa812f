// Flash attention backward as two tcgen05 kernels (head_dim 128), the default backward of attention.cu's forward.
//
//   dkv kernel   one CTA per 128-key tile walks the query tiles that see it, in transposed form so that keys are the
//                TMEM lanes:  S^T = Kh Qh^T,  dP^T = V dO^T,  P^T = exp2(S^T c1 - lse2) masked,  dV += P^T dO,
//                dS^T = P^T (dP^T - delta) scale,  dK += dS^T Qh.
//   dq kernel    one CTA per 128-query tile walks its key tiles (queries are the lanes):  S and dP again, dS, dQ += dS Kh.
//
// P^T, dS^T and dS never touch shared memory: the compute warps write them back to TMEM as packed bf16 pairs over the
// columns of the fp32 tile they were computed from, and the next MMA takes its A operand from TMEM.  Every accumulator
// (dK, dV, dQ) lives in TMEM for the whole CTA: no atomics, no per-tile drain, deterministic results.  Recomputing S and
// dP in the second kernel costs two extra GEMMs per tile pair; in the single-kernel form (attention_bwd.cu) TMEM is full
// and the five GEMMs serialise with the exponentiation and a dQ drain through fp32 atomics.
// Outputs are bf16: dq-hat | dk-hat as [B*T, 2A] for the RoPE / QK-norm backward, dV straight into its third of dqkv.
// Operand views, masking and scaling are those of attention_bwd.cu; the saved log-sum-exp is consumed through a
// pre-pass that also computes delta = rowsum(dO * O).
#include "common.cuh"

namespace bones {

constexpr int ST = 128;
constexpr uint32_t STILE = ST * 128 * 2;   // 32 KB: two 128-byte-swizzled atoms of [128 rows][64 cols]
constexpr uint32_t SATOM = STILE / 2;
constexpr float kLog2e = 1.4426950408889634f;

// Cycle accounting of the dK / dV kernel's roles, compiled in only with -DBONES_ATTN_PROF (a measuring build; the regular
// library carries none of it).  Each role sums the clocks it spends in each of its waits and in its work and stores the
// sums in its CTA's 32 slots of the buffer given to `bones_attn_set_prof`:
//   MMA warp: 0 wait item + K/V  1 wait Q  2 wait dO  3 wait P ready  4 wait accumulators free  5 wait dS ready  6 issue  7 total
//             8 tiles;  compute warp 2: 10 wait statistics  11 wait S  12 P  13 wait dP  14 dS  15 wait done  16 drain  17 total;
//   producer: 20 waits  21 issue.
#ifdef BONES_ATTN_PROF
__device__ long long* g_attn_prof = nullptr;
#define APROF_DECL(n) long long ap_[n] = {}; long long ap_t_ = clock64(); const long long ap_t0_ = ap_t_
#define APROF_ADD(i) do { const long long n_ = clock64(); ap_[i] += n_ - ap_t_; ap_t_ = n_; } while (0)
#define APROF_COUNT(i) (++ap_[i])
#define APROF_STORE(slot, i) do { if (g_attn_prof) g_attn_prof[(long long)blockIdx.x * 32 + (slot)] = ap_[i]; } while (0)
#define APROF_TOTAL(slot) do { if (g_attn_prof) g_attn_prof[(long long)blockIdx.x * 32 + (slot)] = clock64() - ap_t0_; } while (0)
#else
#define APROF_DECL(n)
#define APROF_ADD(i)
#define APROF_COUNT(i)
#define APROF_STORE(slot, i)
#define APROF_TOTAL(slot)
#endif

struct SplitParams {
  int B, T, H;
  float c1, scale;
  int window_tiles;
  const int* doc_start;
  const float2* stats;   // [B, H, T]: (-lse * log2(e), delta)
  __nv_bfloat16* dqk;    // [B*T, 2A]: dq-hat | dk-hat
  __nv_bfloat16* dv;     // rows of dv_ld elements
  long long dv_ld;
  int* err;
  int* items;            // device counter the persistent CTAs of a launch draw their work items from (zero at launch)
};

__device__ __forceinline__ int split_first_tile(const SplitParams& p, int b, int qt) {
  int lo = 0;
  if (p.doc_start) lo = p.doc_start[(long long)b * p.T + qt * ST] / ST;
  if (p.window_tiles > 0) lo = max(lo, qt - p.window_tiles + 1);
  return lo;
}
// Descriptors are the tile's base descriptor plus a compile-time step in the address field (16-byte units; shared-memory
// addresses stay below 2^18, so the field never carries): one 64-bit add per operand and MMA in the issuing loop instead
// of the mask-shift-or chain of a fresh descriptor.
__device__ __forceinline__ uint64_t sdesc_k(uint32_t tile, int k) {   // K-major view, UMMA_K step k
  return umma_smem_desc(tile, 0, 1024, kLayoutSw128) + (uint64_t)(((k >> 2) * SATOM + (k & 3) * 32) >> 4);
}
__device__ __forceinline__ uint64_t sdesc_mn(uint32_t tile, int k) {  // MN-major view of the same bytes
  return umma_smem_desc(tile, SATOM, 1024, kLayoutSw128) + (uint64_t)((k * 2048) >> 4);
}
// Compute warps: four per 32-lane TMEM quadrant, each thread one row and 32 of the tile's 128 columns.  With two per
// quadrant (64 columns a thread) the exponentials and the dS arithmetic of a tile took 3 300 clocks one after the other
// against 2 048 clocks of MMAs; the same work over twice the warps hides a little more of its latency (0.836 -> 0.812 ms
// for the whole backward at B = 16, T = 2048, H = 10).  A P phase still takes about 2 000 clocks: TMEM load, 1 024
// clocks of exponentials on the special-function units, TMEM store, one after the other in every warp at once.
// Computing every other exponential with a cubic on the FMA pipe was measured and made both kernels slower (the
// arithmetic of the dS phase competes for the same issue slots), so all exponentials stay on `ex2.approx`.
constexpr int SCW = 16;                      // compute warps per CTA
constexpr int STHREADS = 64 + 32 * SCW;      // producer warp + MMA warp + compute warps
// TMEM column of UMMA_K step k of a packed bf16 A operand: each compute warp packs its 32 fp32 columns (c0 = 0, 32,
// 64, 96) into the first 16 columns of its own range, two K steps of 8 packed columns each
__device__ __forceinline__ uint32_t packed_col(int k) { return (uint32_t)((k >> 1) * 32 + (k & 1) * 8); }

__device__ __forceinline__ float ex2_fast(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
  return e;
}
// 32 fp32 values -> 16 packed bf16 pairs -> 16 TMEM columns starting at taddr
__device__ __forceinline__ void store_packed32(uint32_t taddr, const float* v) {
  uint32_t pk[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) pk[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
  BONES_TMEM_ST16(taddr, pk);
  tmem_st_wait();
}
// 32 accumulator columns of this thread's row -> 32 bf16 in global memory (two 32-byte sectors)
__device__ __forceinline__ void drain_row32(uint32_t taddr, __nv_bfloat16* dst) {
  uint32_t v[32];
  __syncwarp();
  BONES_TMEM_LD32(taddr, v);
  tmem_ld_wait();
  uint4 u[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    u[g].x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
    u[g].y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
    u[g].z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
    u[g].w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
  }
  st_global_v8(dst, u[0], u[1]);
  st_global_v8(dst + 16, u[2], u[3]);
}

// stats[b,h,t] = (-lse * log2(e), sum_d dO * O); sixteen lanes per (row, head), 16 bytes of each operand per lane.
// Items run in the order of the output, [b, h, t] with t fastest: a group still reads 256 contiguous bytes of each
// operand, and the statistics and the log-sum-exp values of neighbouring groups are neighbours in memory (with the
// head fastest they were T elements apart: one 32-byte sector per 8-byte result).
__global__ void attn_bwd_stats_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ y,
                                      const float* __restrict__ lse, float2* __restrict__ stats, long long M, int T, int H) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const int l16 = threadIdx.x & 15;
  const long long total = M * H;
  const long long it = item < total ? item : total - 1;      // every lane takes part in the shuffles
  const long long bh = it / T;
  const int t = (int)(it - bh * T);
  const long long b = bh / H;
  const int h = (int)(bh - b * H);
  const long long off = ((b * T + t) * H + h) * 128 + l16 * 8;
  const uint4 a = *reinterpret_cast<const uint4*>(dy + off), c = *reinterpret_cast<const uint4*>(y + off);
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = unpack_bf16(aw[i]), fc = unpack_bf16(cw[i]);
    s += fa.x * fc.x + fa.y * fc.y;
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (l16 == 0 && item < total) stats[it] = make_float2(-lse[it] * kLog2e, s);
}

// ---------------------------------------------------------------------------------------------------------------
// dK / dV  (transposed: TMEM lanes are keys, columns are queries).  A Q tile lives from S^T(i) (issued during tile
//          i-1) to dK(i), so Q has a ring of three; dO (with the tile's statistics) is first needed a tile later and
//          has a ring of two.
//          Persistent: one CTA per SM draws (key tile, head, batch) items from a device counter, the key tiles of one
//          (head, batch) side by side.  Barrier phases and the Q / dO rings run on across items; K and V are
//          single-buffered and reloaded as soon as the item's last S^T and dP^T MMAs have been issued, so the next
//          item's first tiles are computed while the compute warps drain dK and dV.
// ---------------------------------------------------------------------------------------------------------------
constexpr uint32_t DKV_STAT = STILE * 7;            // two stages of 128 x (float2 stats), travelling with dO
constexpr uint32_t DKV_BARS = DKV_STAT + 2 * 1024;
constexpr uint32_t DKV_SLACK = 512;                 // room for aligning the tiles to 1024 bytes

__device__ int g_dkv_items;      // item counter of the persistent dK/dV kernel (one launch at a time per device)

struct DkvItem {
  int kt, h, b, n;
};
__device__ __forceinline__ DkvItem dkv_item(const SplitParams& p, int w, int n_tiles) {
  DkvItem it;
  const int grp = w / n_tiles;
  it.kt = w % n_tiles;                                // longest walks (small kt) of a (head, batch) first
  it.h = grp % p.H;
  it.b = grp / p.H;
  int n = 0;
  for (int qt = it.kt; qt < n_tiles; ++qt) {          // the query tiles that see this key tile
    if (split_first_tile(p, it.b, qt) > it.kt) break;
    ++n;
  }
  it.n = n;                                           // >= 1: a key tile is always seen by its own query tile
  return it;
}

__global__ void __launch_bounds__(STHREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_qk, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_dy, const SplitParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  if (base - raw > DKV_SLACK) {                       // the seven tiles would not fit behind the alignment gap
    if (threadIdx.x == 0) atomicCAS(p.err, 0, ERR_WAIT_AUX);
    return;
  }
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sK = base, sV = base + STILE;
  auto sQ = [&](int s) { return base + STILE * (2 + s); };       // three stages
  auto sdO = [&](int s) { return base + STILE * (5 + s); };      // two stages
  const uint32_t bars = base + DKV_BARS;
  enum { B_KV = 0, B_KVFREE, B_Q0, B_Q1, B_Q2, B_QFREE0, B_QFREE1, B_QFREE2, B_DO0, B_DO1, B_DOFREE0, B_DOFREE1, B_SFULL, B_DPFULL,
         B_PREADY, B_DSREADY, B_DONE, B_ACCFREE, B_COUNT };
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t tmem_slot = bars + 8u * B_COUNT;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + DKV_BARS + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + DKV_BARS + 8 * B_COUNT + 8);
  const uint32_t ring_bars = bars + 176u;
  volatile int* ring_slots = reinterpret_cast<volatile int*>(gen + DKV_BARS + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = p.H * 128;
  const int n_tiles = p.T / ST;
  const int total = n_tiles * p.H * p.B;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_KV), 1);
    mbar_init(bar(B_KVFREE), 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(bar(B_Q0 + s), 1);
      mbar_init(bar(B_QFREE0 + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(B_DO0 + s), 1);
      mbar_init(bar(B_DOFREE0 + s), 1);
    }
    mbar_init(bar(B_SFULL), 1);
    mbar_init(bar(B_DPFULL), 1);
    mbar_init(bar(B_PREADY), SCW);
    mbar_init(bar(B_DSREADY), SCW);
    mbar_init(bar(B_DONE), 1);
    mbar_init(bar(B_ACCFREE), SCW);
    for (int s = 0; s < 4; ++s) mbar_init(ring_bars + 8u * s, 1);
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

  // The producer and MMA roles run on all 32 lanes of their warp with warp-uniform state and issue from the elected lane
  // (`elect_one` in common.cuh).  Work items are drawn by lane 0 and handed round with a shuffle.  A lane whose bounded
  // wait ran out turns `dead`: it walks on without waiting or issuing; when lane 0 is dead no further item is drawn.
  if (warp == 0) {
    int g = 0, it = 0;
    bool dead = false;
    APROF_DECL(2);
    for (;; ++it) {
      int w = -1;
      if (lane == 0 && !dead) w = item_publish(ring_bars, ring_slots, it, p.items, total);
      w = warp_uniform(w);
      if (w < 0) break;
      DkvItem im = dkv_item(p, w, n_tiles);
      im.n = warp_uniform(im.n);
      const int row0 = im.b * p.T;
      APROF_ADD(1);
      if (it >= 1 && !dead) dead = !mbar_wait(bar(B_KVFREE), (uint32_t)((it - 1) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
      APROF_ADD(0);
      if (elect_one() && !dead) {
        mbar_arrive_expect_tx(bar(B_KV), 2 * STILE);
        tma_load_2d(sK, &tm_qk, bar(B_KV), A + im.h * 128, row0 + im.kt * ST);
        tma_load_2d(sK + SATOM, &tm_qk, bar(B_KV), A + im.h * 128 + 64, row0 + im.kt * ST);
        tma_load_2d(sV, &tm_v, bar(B_KV), 2 * A + im.h * 128, row0 + im.kt * ST);
        tma_load_2d(sV + SATOM, &tm_v, bar(B_KV), 2 * A + im.h * 128 + 64, row0 + im.kt * ST);
      }
      const float2* stat_row = p.stats + ((long long)im.b * p.H + im.h) * p.T;
      for (int i = 0; i < im.n; ++i, ++g) {
        const int qs = g % 3, ds = g & 1;
        const int r = row0 + (im.kt + i) * ST;
        APROF_ADD(1);
        if (g >= 3 && !dead) dead = !mbar_wait(bar(B_QFREE0 + qs), (uint32_t)(((g - 3) / 3) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
        APROF_ADD(0);
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(bar(B_Q0 + qs), STILE);
          tma_load_2d(sQ(qs), &tm_qk, bar(B_Q0 + qs), im.h * 128, r);
          tma_load_2d(sQ(qs) + SATOM, &tm_qk, bar(B_Q0 + qs), im.h * 128 + 64, r);
        }
        APROF_ADD(1);
        if (g >= 2 && !dead) dead = !mbar_wait(bar(B_DOFREE0 + ds), (uint32_t)(((g - 2) >> 1) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
        APROF_ADD(0);
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(bar(B_DO0 + ds), STILE + 1024);
          tma_load_2d(sdO(ds), &tm_dy, bar(B_DO0 + ds), im.h * 128, r);
          tma_load_2d(sdO(ds) + SATOM, &tm_dy, bar(B_DO0 + ds), im.h * 128 + 64, r);
          bulk_load(base + DKV_STAT + ds * 1024, stat_row + (im.kt + i) * ST, 1024, bar(B_DO0 + ds));
        }
      }
    }
    APROF_ADD(1);
    if (lane == 0) { APROF_STORE(20, 0); APROF_STORE(21, 1); }
  } else if (warp == 1) {
    const uint32_t id_kk = umma_idesc_f16(128, 128, 1, 0, 0);
    const uint32_t id_km = umma_idesc_f16(128, 128, 1, 0, 1);
    bool dead = false;
    APROF_DECL(8);
    auto issue_s = [&](int t) {                           // S^T(t) = Kh Qh(t)^T
      APROF_ADD(6);
      if (!dead) dead = !mbar_wait(bar(B_Q0 + t % 3), (uint32_t)((t / 3) & 1), abort_flag, p.err, ERR_WAIT_FULL);
      APROF_ADD(1);
      tc_fence_after();
      if (elect_one() && !dead) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tS, sdesc_k(sK, k), sdesc_k(sQ(t % 3), k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_SFULL));
      }
    };
    auto issue_dp = [&](int t, bool last) {               // dP^T(t) = V dO(t)^T; after the item's last one K and V are free
      APROF_ADD(6);
      if (!dead) dead = !mbar_wait(bar(B_DO0 + (t & 1)), (uint32_t)((t >> 1) & 1), abort_flag, p.err, ERR_WAIT_FULL);
      APROF_ADD(2);
      tc_fence_after();
      if (elect_one() && !dead) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdP, sdesc_k(sV, k), sdesc_k(sdO(t & 1), k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_DPFULL));
        if (last) tc_commit(bar(B_KVFREE));
      }
    };
    int g = 0, it = 0;
    for (;; ++it) {
      int w = -1;
      APROF_ADD(6);
      if (!dead) w = item_take(ring_bars, ring_slots, it, abort_flag, p.err);
      w = warp_uniform(w);
      if (w < 0) break;
      DkvItem im = dkv_item(p, w, n_tiles);
      im.n = warp_uniform(im.n);
      if (!dead) dead = !mbar_wait(bar(B_KV), (uint32_t)(it & 1), abort_flag, p.err, ERR_WAIT_FULL);
      APROF_ADD(0);
      // the first tile's S^T and dP^T go behind the previous item's last dV / dK MMAs on the same (in-order) pipe
      issue_s(g);
      issue_dp(g, im.n == 1);
      for (int i = 0; i < im.n; ++i, ++g) {
        const int s = g & 1, qs = g % 3;
        const uint32_t ph = (uint32_t)(g & 1);
        const bool more = i + 1 < im.n;
        // P^T(g) sits packed in the S^T columns: dV += P^T dO, then S^T(g+1) behind it
        APROF_ADD(6);
        APROF_COUNT(7);
        if (!dead) dead = !mbar_wait(bar(B_PREADY), ph, abort_flag, p.err, ERR_WAIT_AUX);
        APROF_ADD(3);
        // the previous item's dK / dV must have been drained
        if (i == 0 && it >= 1 && !dead) dead = !mbar_wait(bar(B_ACCFREE), (uint32_t)((it - 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        APROF_ADD(4);
        tc_fence_after();
        if (elect_one() && !dead) {
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16_ts(tdV, tS + packed_col(k), sdesc_mn(sdO(s), k), id_km, (i | k) ? 1u : 0u);
        }
        if (more) issue_s(g + 1);
        // dS^T(g) sits packed in the dP^T columns: dK += dS^T Qh, then dP^T(g+1) behind it
        APROF_ADD(6);
        if (!dead) dead = !mbar_wait(bar(B_DSREADY), ph, abort_flag, p.err, ERR_WAIT_AUX);
        APROF_ADD(5);
        tc_fence_after();
        if (elect_one() && !dead) {
#pragma unroll
          for (int k = 0; k < 8; ++k) umma_f16_ts(tdK, tdP + packed_col(k), sdesc_mn(sQ(qs), k), id_km, (i | k) ? 1u : 0u);
          tc_commit(bar(B_QFREE0 + qs));
          tc_commit(bar(B_DOFREE0 + s));     // dO(g) was read by dV(g); its statistics were in use until dS(g) was stored
          if (!more) tc_commit(bar(B_DONE));
        }
        if (more) issue_dp(g + 1, i + 2 == im.n);
      }
    }
    APROF_ADD(6);
    if (lane == 0) {
      for (int i = 0; i < 7; ++i) APROF_STORE(i, i);
      APROF_TOTAL(7);
      APROF_STORE(8, 7);
    }
  } else {
    const int q = warp & 3, part = (warp - 2) >> 2;
    const int r = q * 32 + lane;                       // key row of this thread
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int c0 = part * 32;                          // first query column of this thread
    bool ok = true;
    int g = 0, it = 0;
    APROF_DECL(8);
    for (;; ++it) {
      const int w = ok ? item_take(ring_bars, ring_slots, it, abort_flag, p.err) : -1;
      if (w < 0) break;
      const DkvItem im = dkv_item(p, w, n_tiles);
      const int k0 = im.kt * ST, kpos = k0 + r, row0 = im.b * p.T;
      int nx_lo_last = p.doc_start ? p.doc_start[(long long)im.b * p.T + im.kt * ST + ST - 1] : 0;
      for (int i = 0; i < im.n; ++i, ++g) {
        const int s = g & 1;
        const uint32_t ph = (uint32_t)(g & 1);
        APROF_ADD(2);
        bool got = mbar_wait(bar(B_DO0 + s), (uint32_t)((g >> 1) & 1), abort_flag, p.err, ERR_WAIT_FULL);   // this tile's statistics
        APROF_ADD(0);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        const float4* st4 = reinterpret_cast<const float4*>(gen + DKV_STAT + s * 1024) + c0 / 2;   // two queries per float4
        // document starts of this tile's queries (global, cached): only the tile that straddles a document start past
        // this key tile needs them element by element, and its last query decides that
        const int* slo = p.doc_start ? p.doc_start + (long long)im.b * p.T + (im.kt + i) * ST : nullptr;
        const bool need_doc = slo && nx_lo_last > k0;
        if (slo && i + 1 < im.n) nx_lo_last = slo[2 * ST - 1];
        float pr[32];
        got = mbar_wait(bar(B_SFULL), ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
        APROF_ADD(1);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        {
          uint32_t v0[32];
          __syncwarp();
          BONES_TMEM_LD32(tS + lane_addr + (uint32_t)c0, v0);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float4 a = st4[j];
            pr[2 * j] = ex2_fast(fmaf(__uint_as_float(v0[2 * j]), p.c1, a.x));
            pr[2 * j + 1] = ex2_fast(fmaf(__uint_as_float(v0[2 * j + 1]), p.c1, a.z));
          }
        }
        if (i == 0) {                                    // diagonal tile: a key sees only queries at or after it
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (r > c0 + j) pr[j] = 0.f;
        }
        if (need_doc) {                                  // a query sees only keys of its own document
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (kpos < slo[c0 + j]) pr[j] = 0.f;
        }
        store_packed32(tS + lane_addr + (uint32_t)c0, pr);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_PREADY));
        APROF_ADD(2);
        got = mbar_wait(bar(B_DPFULL), ph, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
        APROF_ADD(3);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        {
          uint32_t v0[32];
          __syncwarp();
          BONES_TMEM_LD32(tdP + lane_addr + (uint32_t)c0, v0);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float4 a = st4[j];
            pr[2 * j] *= (__uint_as_float(v0[2 * j]) - a.y) * p.scale;
            pr[2 * j + 1] *= (__uint_as_float(v0[2 * j + 1]) - a.w) * p.scale;
          }
        }
        store_packed32(tdP + lane_addr + (uint32_t)c0, pr);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_DSREADY));
        APROF_ADD(4);
      }
      if (!ok) break;
      const bool got = mbar_wait(bar(B_DONE), (uint32_t)(it & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      APROF_ADD(5);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      drain_row32(tdK + lane_addr + (uint32_t)c0, p.dqk + ((long long)(row0 + kpos)) * 2 * A + A + (long long)im.h * 128 + c0);
      drain_row32(tdV + lane_addr + (uint32_t)c0, p.dv + ((long long)(row0 + kpos)) * p.dv_ld + (long long)im.h * 128 + c0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_ACCFREE));
      APROF_ADD(6);
    }
    if (warp == 2 && lane == 0) {
      APROF_STORE(10, 0); APROF_STORE(11, 1); APROF_STORE(12, 2); APROF_STORE(13, 3); APROF_STORE(14, 4); APROF_STORE(15, 5); APROF_STORE(16, 6);
      APROF_TOTAL(17);
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
// dQ  (TMEM lanes are queries, columns are keys; dP double-buffered so the MMAs of tile j+1 run under the
//      exponentiation of tile j).  K tiles live from S(j) to dQ(j), V tiles only until dP(j): a K ring of three and a V
//      ring of two keep every load a full tile ahead of its first use.
//      One "dS ready" barrier per dP buffer: S(j+1) and dP(j+1) are issued before dS(j) is awaited, so a compute warp
//      can finish tile j+1 while a slower one is still on tile j; with one barrier for both buffers its second
//      arrival completed the slower warp's phase and the dQ MMAs read that warp's columns before it had stored them
//      (a few non-finite rows of dq once in a few hundred calls, more often with sixteen compute warps whose masking
//      work differs).  dP(j+2) is only issued after dQ(j), so nobody can be two tiles ahead.
//      Persistent: one CTA per SM walks (query tile, head, batch) items in the forward kernel's order (the query tiles
//      of one (head, batch) run at the same time and share K/V through L2).  Barrier phases, the K/V rings and the dP
//      buffers run on across items; Q and dO are single-buffered and reloaded as soon as the item's last S and dP MMAs
//      have been issued, so the next item's first tiles are computed while the compute warps drain dQ.
// ---------------------------------------------------------------------------------------------------------------
constexpr uint32_t DQ_BARS = STILE * 7;

__device__ int g_dq_items;       // item counter of the persistent dQ kernel (one launch at a time per device)

struct DqItem {
  int qt, h, b, kt0, n;
};
__device__ __forceinline__ DqItem dq_item(const SplitParams& p, int w, int n_tiles) {
  DqItem it;
  const int grp = w / n_tiles;
  it.qt = n_tiles - 1 - (w % n_tiles + grp) % n_tiles;
  it.h = grp % p.H;
  it.b = grp / p.H;
  it.kt0 = split_first_tile(p, it.b, it.qt);
  it.n = it.qt - it.kt0 + 1;
  return it;
}

__global__ void __launch_bounds__(STHREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qk, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_dy, const SplitParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sQ = base, sdO = base + STILE;
  auto sK = [&](int s) { return base + STILE * (2 + s); };      // three stages
  auto sV = [&](int s) { return base + STILE * (5 + s); };      // two stages
  const uint32_t bars = base + DQ_BARS;
  enum { B_QDO = 0, B_QDOFREE, B_K0, B_K1, B_K2, B_KFREE0, B_KFREE1, B_KFREE2, B_V0, B_V1, B_VFREE0, B_VFREE1, B_SFULL, B_SFREE,
         B_DPFULL0, B_DPFULL1, B_DSREADY0, B_DSREADY1, B_DONE, B_DQFREE, B_COUNT };
  auto bar = [&](int i) { return bars + 8u * i; };
  const uint32_t tmem_slot = bars + 8u * B_COUNT;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + DQ_BARS + 8 * B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + DQ_BARS + 8 * B_COUNT + 8);
  const uint32_t ring_bars = bars + 176u;
  volatile int* ring_slots = reinterpret_cast<volatile int*>(gen + DQ_BARS + 208);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int A = p.H * 128;
  const int n_tiles = p.T / ST;
  const int total = n_tiles * p.H * p.B;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QDO), 1);
    mbar_init(bar(B_QDOFREE), 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(bar(B_K0 + s), 1);
      mbar_init(bar(B_KFREE0 + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(B_V0 + s), 1);
      mbar_init(bar(B_VFREE0 + s), 1);
      mbar_init(bar(B_DPFULL0 + s), 1);
    }
    mbar_init(bar(B_SFULL), 1);
    mbar_init(bar(B_SFREE), SCW);
    mbar_init(bar(B_DSREADY0), SCW);
    mbar_init(bar(B_DSREADY1), SCW);
    mbar_init(bar(B_DONE), 1);
    mbar_init(bar(B_DQFREE), SCW);
    for (int s = 0; s < 4; ++s) mbar_init(ring_bars + 8u * s, 1);
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
  const uint32_t tS = tmem, tdQ = tmem + 384;
  auto tdP = [&](int s) { return tmem + 128u + (uint32_t)s * 128u; };

  // producer and MMA roles: warp-uniform loops issuing from the elected lane, as in the dK / dV kernel above
  if (warp == 0) {
    int g = 0, it = 0;
    bool dead = false;
    for (;; ++it) {
      int w = -1;
      if (lane == 0 && !dead) w = item_publish(ring_bars, ring_slots, it, p.items, total);
      w = warp_uniform(w);
      if (w < 0) break;
      DqItem im = dq_item(p, w, n_tiles);
      im.kt0 = warp_uniform(im.kt0);
      im.n = im.qt - im.kt0 + 1;
      const int row0 = im.b * p.T, rq = row0 + im.qt * ST;
      if (it >= 1 && !dead) dead = !mbar_wait(bar(B_QDOFREE), (uint32_t)((it - 1) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
      if (elect_one() && !dead) {
        mbar_arrive_expect_tx(bar(B_QDO), 2 * STILE);
        tma_load_2d(sQ, &tm_qk, bar(B_QDO), im.h * 128, rq);
        tma_load_2d(sQ + SATOM, &tm_qk, bar(B_QDO), im.h * 128 + 64, rq);
        tma_load_2d(sdO, &tm_dy, bar(B_QDO), im.h * 128, rq);
        tma_load_2d(sdO + SATOM, &tm_dy, bar(B_QDO), im.h * 128 + 64, rq);
      }
      for (int j = 0; j < im.n; ++j, ++g) {
        const int ks = g % 3, vs = g & 1;
        const int r = row0 + (im.kt0 + j) * ST;
        if (g >= 3 && !dead) dead = !mbar_wait(bar(B_KFREE0 + ks), (uint32_t)(((g - 3) / 3) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(bar(B_K0 + ks), STILE);
          tma_load_2d(sK(ks), &tm_qk, bar(B_K0 + ks), A + im.h * 128, r);
          tma_load_2d(sK(ks) + SATOM, &tm_qk, bar(B_K0 + ks), A + im.h * 128 + 64, r);
        }
        if (g >= 2 && !dead) dead = !mbar_wait(bar(B_VFREE0 + vs), (uint32_t)(((g - 2) >> 1) & 1), abort_flag, p.err, ERR_WAIT_EMPTY);
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(bar(B_V0 + vs), STILE);
          tma_load_2d(sV(vs), &tm_v, bar(B_V0 + vs), 2 * A + im.h * 128, r);
          tma_load_2d(sV(vs) + SATOM, &tm_v, bar(B_V0 + vs), 2 * A + im.h * 128 + 64, r);
        }
      }
    }
  } else if (warp == 1) {
    const uint32_t id_kk = umma_idesc_f16(128, 128, 1, 0, 0);
    const uint32_t id_km = umma_idesc_f16(128, 128, 1, 0, 1);
    bool dead = false;
    // S(t) and dP(t) of running tile t; `last`: t is the last tile of its item, after which Q and dO may be reloaded
    auto issue_sdp = [&](int t, bool last) {
      if (!dead) dead = !mbar_wait(bar(B_K0 + t % 3), (uint32_t)((t / 3) & 1), abort_flag, p.err, ERR_WAIT_FULL);
      if (t >= 1 && !dead) dead = !mbar_wait(bar(B_SFREE), (uint32_t)((t - 1) & 1), abort_flag, p.err, ERR_WAIT_AUX);
      tc_fence_after();
      if (elect_one() && !dead) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tS, sdesc_k(sQ, k), sdesc_k(sK(t % 3), k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_SFULL));
      }
      if (!dead) dead = !mbar_wait(bar(B_V0 + (t & 1)), (uint32_t)((t >> 1) & 1), abort_flag, p.err, ERR_WAIT_FULL);
      tc_fence_after();
      // dP(t) goes into the buffer whose packed dS(t-2) the dQ MMAs of tile t-2 (issued earlier, same pipe) have read
      if (elect_one() && !dead) {
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16(tdP(t & 1), sdesc_k(sdO, k), sdesc_k(sV(t & 1), k), id_kk, k ? 1u : 0u);
        tc_commit(bar(B_DPFULL0 + (t & 1)));
        tc_commit(bar(B_VFREE0 + (t & 1)));
        if (last) tc_commit(bar(B_QDOFREE));
      }
    };
    int g = 0, it = 0;
    for (;; ++it) {
      int w = -1;
      if (!dead) w = item_take(ring_bars, ring_slots, it, abort_flag, p.err);
      w = warp_uniform(w);
      if (w < 0) break;
      DqItem im = dq_item(p, w, n_tiles);
      im.kt0 = warp_uniform(im.kt0);
      im.n = im.qt - im.kt0 + 1;
      if (!dead) dead = !mbar_wait(bar(B_QDO), (uint32_t)(it & 1), abort_flag, p.err, ERR_WAIT_FULL);
      for (int j = 0; j < im.n; ++j, ++g) {
        if (j == 0) issue_sdp(g, im.n == 1);
        if (j + 1 < im.n) issue_sdp(g + 1, j + 2 == im.n);
        // dS(g) sits packed in the dP(g) columns: dQ += dS Kh(g), which also frees that K stage
        if (!dead) dead = !mbar_wait(bar(B_DSREADY0 + (g & 1)), (uint32_t)((g >> 1) & 1), abort_flag, p.err, ERR_WAIT_AUX);
        if (j == 0 && it >= 1 && !dead) dead = !mbar_wait(bar(B_DQFREE), (uint32_t)((it - 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        if (elect_one() && !dead) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_f16_ts(tdQ, tdP(g & 1) + packed_col(k), sdesc_mn(sK(g % 3), k), id_km, (j | k) ? 1u : 0u);
          tc_commit(bar(B_KFREE0 + g % 3));
          if (j + 1 == im.n) tc_commit(bar(B_DONE));
        }
      }
    }
  } else {
    const int q = warp & 3, part = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int c0 = part * 32;
    bool ok = true;
    int g = 0, it = 0;
    for (;; ++it) {
      const int w = ok ? item_take(ring_bars, ring_slots, it, abort_flag, p.err) : -1;
      if (w < 0) break;
      const DqItem im = dq_item(p, w, n_tiles);
      const int qpos = im.qt * ST + r, row0 = im.b * p.T;
      const float2 st = p.stats[((long long)im.b * p.H + im.h) * p.T + qpos];
      int lo = 0;
      if (p.doc_start) lo = p.doc_start[(long long)im.b * p.T + qpos];
      for (int j = 0; j < im.n; ++j, ++g) {
        const int s = g & 1;
        bool got = mbar_wait(bar(B_SFULL), (uint32_t)(g & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        const int k0 = (im.kt0 + j) * ST + c0;
        const bool need_mask = __any_sync(0xffffffffu, (k0 + 31 > qpos) || (k0 < lo));
        float pr[32];
        {
          uint32_t v0[32];
          __syncwarp();
          BONES_TMEM_LD32(tS + lane_addr + (uint32_t)c0, v0);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_SFREE));
#pragma unroll
          for (int i = 0; i < 32; ++i) pr[i] = ex2_fast(fmaf(__uint_as_float(v0[i]), p.c1, st.x));
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kp = k0 + i;
            if (kp > qpos || kp < lo) pr[i] = 0.f;
          }
        }
        got = mbar_wait(bar(B_DPFULL0 + s), (uint32_t)((g >> 1) & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        {
          uint32_t v0[32];
          __syncwarp();
          BONES_TMEM_LD32(tdP(s) + lane_addr + (uint32_t)c0, v0);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) pr[i] *= (__uint_as_float(v0[i]) - st.y) * p.scale;
        }
        store_packed32(tdP(s) + lane_addr + (uint32_t)c0, pr);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_DSREADY0 + s));
      }
      if (!ok) break;
      const bool got = mbar_wait(bar(B_DONE), (uint32_t)(it & 1), abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      drain_row32(tdQ + lane_addr + (uint32_t)c0, p.dqk + ((long long)(row0 + qpos)) * 2 * A + (long long)im.h * 128 + c0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_DQFREE));
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

// stats: [B, H, T] float2 scratch filled by the pre-pass
int bones_attn_bwd_stats(const void* dy, const void* y, const float* lse, void* stats, long long M, int T, int H, void* stream) {
  const long long threads = M * H * 16;
  attn_bwd_stats_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)y,
                                                                                       lse, (float2*)stats, M, T, H);
  return (int)cudaGetLastError();
}

// qk: [B*T, 2A] rotated, normalised q | k;  qkv: [B*T, 3A] (values read in place);  dy: [B*T, A];  stats from the pre-pass.
// Outputs (bf16, every element overwritten): dqk [B*T, 2A];  dv rows of dv_ld elements (e.g. the last third of dqkv).
int bones_attn_bwd_split(const void* qk, const void* qkv, const void* dy, const void* stats, void* dqk, void* dv, long long dv_ld,
                         const int* doc_start, int B, int T, int H, float scale, int window_tiles, void* stream) {
  if (T % ST) return -2;
  if ((dv_ld % 16) || ((uintptr_t)dv & 31) || ((uintptr_t)dqk & 31) || ((uintptr_t)stats & 15) ||
      (doc_start && ((uintptr_t)doc_start & 15)))
    return -3;
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
  p.c1 = scale * kLog2e;
  p.scale = scale;
  p.window_tiles = window_tiles;
  p.doc_start = doc_start;
  p.stats = (const float2*)stats;
  p.dqk = (__nv_bfloat16*)dqk;
  p.dv = (__nv_bfloat16*)dv;
  p.dv_ld = dv_ld;
  p.err = error_word();
  constexpr size_t smem_dkv = (size_t)DKV_BARS + 256 + DKV_SLACK;
  constexpr size_t smem_dq = (size_t)DQ_BARS + 256 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv));
    BONES_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq));
    attr_done = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev < 0 || dev >= 64) return -2;
  const long long items = (long long)(T / ST) * H * B;
  const unsigned grid = (unsigned)(items < sms ? items : sms);          // persistent: one CTA per SM in both kernels
  static int* counter_dkv[64] = {};
  static int* counter_dq[64] = {};
  if (!counter_dkv[dev]) BONES_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&counter_dkv[dev]), g_dkv_items));
  if (!counter_dq[dev]) BONES_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&counter_dq[dev]), g_dq_items));
  BONES_CHECK(cudaMemsetAsync(counter_dkv[dev], 0, sizeof(int), s));
  BONES_CHECK(cudaMemsetAsync(counter_dq[dev], 0, sizeof(int), s));
  p.items = counter_dkv[dev];
  attn_bwd_dkv_kernel<<<grid, STHREADS, smem_dkv, s>>>(tq, tv, td, p);
  BONES_CHECK(cudaGetLastError());
  p.items = counter_dq[dev];
  attn_bwd_dq_kernel<<<grid, STHREADS, smem_dq, s>>>(tq, tv, td, p);
  return (int)cudaGetLastError();
}

#ifdef BONES_ATTN_PROF
// measuring build: device buffer of 32 counters per CTA that the next dK / dV launches fill (null switches it off)
void bones_attn_set_prof(void* buf) {
  long long* b = (long long*)buf;
  cudaMemcpyToSymbol(bones::g_attn_prof, &b, sizeof(b));
}
#endif
}  // extern "C"
