// MXFP8 block-scaled GEMM on CTA pairs: `tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale`, 256 x BN output tiles.
//
//   D[b] = epilogue( alpha * (A_q 2^sfa)[b] * (B_q 2^sfb)[b]^T , R[b] )        A: logical [M, K]   B: logical [N, K]
//
// Elements are E4M3, one UE8M0 scale per 32 elements of K (OCP microscaling).  Either operand may be K-major (K
// contiguous: forward and input-gradient GEMMs) or MN-major (the M / N index contiguous: the weight-gradient GEMM
// `dW = dY^T X` contracts over tokens and reads both activations as stored, quantised along the token axis).
//
// Why pairs: an fp8 MMA retires twice the flops of a bf16 one per operand byte the SM has to pull out of L2.  A single
// CTA with a 128 x 160 tile needs about 115 bytes per clock from L2 at full tensor rate and is bound by that path at
// half of it.  In a pair each CTA loads its own 128 rows of A and only half of the B tile; both tensor cores read both
// halves through the cluster's shared-memory window, which cuts the demand to 64-83 bytes per clock.
//
// Tile N (`bn`, a run-time argument): 160 or 224 with two accumulators in TMEM (the epilogue of a tile overlaps the MMAs
// of the next), or 256 with one (weight gradients: the contraction is tens of thousands long, the epilogue a few per
// cent).  TMEM columns: accumulators from 0, four rotating sets of scale columns from 464.
//
// Scales in global memory are 512-byte chunks, one per (128 rows, 128 of K), in the image `tcgen05.cp.32x128b.warpx4`
// spreads over four TMEM columns: byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (k % 128) / 32.  Chunks of an operand
// with `group` rows per tile (128 for A, `bn` for B) are ordered [row group][K block][chunk in group], so the scales of
// one tile and K block are one contiguous run (512 bytes for A, 1024 for B) fetched by one TMA copy into each CTA's own
// shared memory; the leader's `tcgen05.cp.cta_group::2` then moves them into both CTAs' TMEM.
//
// Epilogues: bf16 / residual / ReLU^2 / ReLU^2-backward (acc * 2 sqrt(h)) / fp32 accumulate (split-K, vector atomics).
// The first four can also emit the result re-quantised to MXFP8 -- along N (each thread owns 32 consecutive columns of
// its row: one block of the next GEMM's K axis) and along M (32 consecutive rows are the 32 lanes of a warp: one
// `redux.sync.max` per column gives every lane the block maximum) -- so a chain c_fc -> ReLU^2 -> c_proj and its
// backward never re-read bf16 activations to quantise them, and the weight-gradient GEMMs find their token-axis
// operands ready.
//
// Protocol (every wait bounded, see common.cuh) as in gemm_bf16_2cta.cu: each CTA's producer thread issues its TMA loads
// in the `.cta_group::2` form that credits the leader's `full[s]`; the leader's MMA thread copies the scales, issues the
// pair MMAs and commits with `.multicast::cluster` to `empty[s]` / `tmem_full[a]` of both CTAs; sixteen epilogue warps
// per CTA (the quantising epilogues are instruction-bound: eight warps took 2.4 times the MMA time of a K = 1280 tile)
// drain their 128 rows and arrive on the leader's `tmem_empty[a]`.  No TMA load uses cluster multicast.
//
// Reference counterparts: fp8 fused MLP forward / backward (round2/source/kernels/nki_mlp_fused8.py:508-570), fp8
// projections (nki_attn_tt8g.py:616-623) and the fp8 weight-gradient GEMM (nki_dw8.py:239); per-block scales replace
// their per-tensor power-of-two scales.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace bones {

struct Mx2Params {
  int M, N, K, batch;
  int a_major, b_major;
  int bn;                       // pair tile N
  int acc_stages;               // 2 (bn <= 224) or 1
  int epi;                      // GemmEpi numbering: 0 bf16, 1 + beta*R, 2 ReLU^2, 3 fp32 +=, 4 * 2 sqrt(R)
  float alpha, beta;
  void* D;                      // bf16 (fp32 with epi 3); may be null when only quantised outputs are wanted
  long long ldd, strideD;
  const void* R;
  long long ldr, strideR;
  uint8_t* Dq;                  // optional [batch, M, N] E4M3, quantised along N ...
  uint8_t* Dsf;                 // ... with scale chunks of an operand with `dq_group` rows per tile and K = N
  int dq_group;
  long long dsf_batch;          // bytes between batches of Dsf
  uint8_t* Dt;                  // optional [batch, M, N] E4M3, quantised along M ...
  uint8_t* Dtsf;                // ... with scale chunks of an operand with rows = N, `dt_group` rows per tile, K = M
  int dt_group;
  long long dtsf_batch;
  int sfa_rows_per_batch;       // rows of the [*, 256] scale maps per batch
  int sfb_rows_per_batch;
  int* err;
  int tiles_m, tiles_n;
  int splits, atomic, wide;
  int sf_sets;                  // copies of the scale columns in TMEM that the K blocks rotate through (1, 2 or 4)
  int sf_warp;                  // 1: a warp of its own issues the scale copies, ahead of the MMA thread
  int staged;                   // 1: bf16 / E4M3 outputs are turned round through the staging tiles (five stages)
  long long* prof;              // BONES_MX_PROF builds only: 32 cycle counters per CTA (null otherwise)
};

// Cycle accounting of the roles, compiled in only with -DBONES_MX_PROF (a measuring build; the regular library carries
// none of it).  Each role thread sums the clocks it spends in each of its waits and in issuing, and stores the sums in
// its CTA's 32 slots of `prof` on the way out:
//   0 MMA: wait accumulator free   1 MMA: wait stage full   2 MMA: wait scales copied   3 MMA: issue   4 MMA: total
//   5 producer: wait stage empty   6 producer: issue        7 producer: total
//   8 scale copy: wait stage full  9 scale copy: wait columns free   10 scale copy: issue
//   11 epilogue warp 3: wait accumulator full   12 epilogue warp 3: drain   13 epilogue warp 3: total   14 K blocks   15 tiles
//   16 MMA: the MMA instructions and commits of a block
//   epilogue warp 3, staged epilogue, per phase: 19 TMEM load  20 wait for the previous TMA store  21 auxiliary operand + maths + bf16 tile
//   + copy along N  22 copy along M  23 fence + read-back + stores  24 chunks
#ifdef BONES_MX_PROF
#define QPROF_DECL(n) long long qp_[n] = {}; long long qp_t_ = clock64(); const long long qp_t0_ = qp_t_
#define QPROF_ADD(i) do { const long long n_ = clock64(); qp_[i] += n_ - qp_t_; qp_t_ = n_; } while (0)
#define QPROF_COUNT(i) (++qp_[i])
#define QPROF_STORE(slot, i) do { if (p.prof) p.prof[(long long)blockIdx.x * 32 + (slot)] = qp_[i]; } while (0)
#define QPROF_TOTAL(slot) do { if (p.prof) p.prof[(long long)blockIdx.x * 32 + (slot)] = clock64() - qp_t0_; } while (0)
#define QEPI_ARG , long long* qe_, long long& qe_t_
#define QEPI_PASS , qe_, qe_t_
#define QEPI_ADD(i) do { const long long n_ = clock64(); qe_[i] += n_ - qe_t_; qe_t_ = n_; } while (0)
#else
#define QEPI_ARG
#define QEPI_PASS
#define QEPI_ADD(i)
#define QPROF_DECL(n)
#define QPROF_ADD(i)
#define QPROF_COUNT(i)
#define QPROF_STORE(slot, i)
#define QPROF_TOTAL(slot)
#endif

constexpr int QM = 256, QK = 128, QSTAGES = 6;          // stages: 6, or 5 with the epilogue's staging tiles behind them
constexpr int QSTAGES_STAGED = 5;
constexpr uint32_t QA_BYTES = 128 * QK;            // 16384
constexpr uint32_t QB_BYTES = 128 * QK;            // up to 128 rows (K-major: bn / 2 rows; MN-major: 128 K rows)
constexpr uint32_t QSFA_BYTES = 512, QSFB_BYTES = 1024;
constexpr uint32_t QSTAGE_STRIDE = 34816;          // 34 KB >= 16384 + 16384 + 512 + 1024, tiles stay 1024-aligned
// scale columns: up to four sets of (A: 4 columns, B: 8 columns) from column 464.  With one set the `tcgen05.cp` of a K
// block has to wait for the MMAs of the block before (they read the columns it overwrites) and the MMAs for the copy:
// the tensor pipe idles for the copies' latency every 128 of K.  Rotating sets removes the first wait.
constexpr uint32_t QTMEM_SF0 = 464, QTMEM_SF_STRIDE = 12;
constexpr int kGroupMq = 8;
constexpr int kSfSetsMax = 4;
constexpr int kNumBars = 2 * QSTAGES + 4 + 2 * kSfSetsMax;
// Epilogue staging behind the stages: per epilogue warp one 32 x 32 bf16 tile (64-byte swizzle), two 32 x 32 E4M3 tiles
// (32-byte swizzle) and, behind all of them, 32 floats of scratch per warp.
constexpr int kEpiWarpsQ = 12;
constexpr uint32_t QSTG_D = 0, QSTG_Q = 2048, QSTG_T = 3072, QSTG_BYTES = 4096, QSTG_SCRATCH = 128;
constexpr uint32_t QSTG_BASE = QSTAGES_STAGED * QSTAGE_STRIDE;
constexpr uint32_t QSCRATCH_BASE = QSTG_BASE + kEpiWarpsQ * QSTG_BYTES;
constexpr uint32_t QBARS_BASE = QSCRATCH_BASE + kEpiWarpsQ * QSTG_SCRATCH;
static_assert(QBARS_BASE >= QSTAGES * QSTAGE_STRIDE, "the barriers sit behind both layouts");
constexpr size_t QSMEM_BYTES = (size_t)QBARS_BASE + 8 * kNumBars + 16 + 1024;

__device__ __forceinline__ void decode_tile_q(int tile, int tiles_m, int tiles_n, int& b, int& mb, int& nb) {
  const int per_batch = tiles_m * tiles_n;
  b = tile / per_batch;
  const int rem = tile - b * per_batch;
  const int group_size = kGroupMq * tiles_n;
  const int gid = rem / group_size;
  const int first_m = gid * kGroupMq;
  const int gsz = min(tiles_m - first_m, kGroupMq);
  const int in_group = rem - gid * group_size;
  mb = first_m + in_group % gsz;
  nb = in_group / gsz;
}

__device__ __forceinline__ uint32_t q_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void q_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void q_mbar_arrive_cluster(uint32_t local_bar, uint32_t cta) {
  asm volatile(
      "{\n"
      ".reg .b32 rem;\n"
      "mapa.shared::cluster.u32 rem, %0, %1;\n"
      "mbarrier.arrive.shared::cluster.b64 _, [rem];\n"
      "}\n" ::"r"(local_bar),
      "r"(cta)
      : "memory");
}
// Pair-mode TMA loads: the destination is this CTA's shared memory, the transaction bytes go to the leader's barrier.
__device__ __forceinline__ void q_tma_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & 0xFEFFFFFFu), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void q_tma_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & 0xFEFFFFFFu), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void q_umma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// shared -> TMEM copy of 32 lanes x 128 bits, replicated to the four sub-partitions, in both CTAs of the pair (each from
// its own shared memory at the descriptor's offset)
__device__ __forceinline__ void q_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// commit that arrives on a barrier of the issuing (leader) CTA only
__device__ __forceinline__ void q_commit_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void q_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
               : "memory");
}

// smallest power of two 2^e with amax / 2^e <= 448 = 1.75 * 2^8; returns 2^-e and the biased exponent
__device__ __forceinline__ float q_scale_pow2(float amax, int& biased) {
  if (!(amax > 0.f)) { biased = 0; return 0.f; }
  const uint32_t bits = __float_as_uint(amax);
  int e = (int)((bits >> 23) & 0xff) - 127 - 8;
  if ((bits & 0x7fffffu) > 0x600000u) e += 1;
  e = max(-127, min(127, e));
  biased = e + 127;
  return __uint_as_float((uint32_t)(127 - e) << 23);
}
__device__ __forceinline__ uint32_t q_pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
// byte offset of the scale of (row r, contraction index k) in an operand with `kblocks` K blocks of 128 and `group` rows
// per tile
__device__ __host__ __forceinline__ size_t q_sf_offset(long long r, long long k, long long kblocks, int group) {
  const long long g = r / group, t = r - g * group;
  const int chunks = (group + 127) >> 7;
  return (size_t)(((g * kblocks + (k >> 7)) * chunks + (t >> 7)) * 512 + (t & 31) * 16 + ((t & 127) >> 5) * 4 + ((k & 127) >> 5));
}

// scale-chunk offset with 32-bit arithmetic; `shift` >= 0 when the tile height is a power of two
__device__ __forceinline__ uint32_t q_sf_offset32(uint32_t r, uint32_t k, uint32_t kblocks, int group, int shift) {
  const uint32_t g = shift >= 0 ? (r >> shift) : r / (uint32_t)group;
  const uint32_t t = r - g * (uint32_t)group;
  const uint32_t chunks = ((uint32_t)group + 127u) >> 7;
  return ((g * kblocks + (k >> 7)) * chunks + (t >> 7)) * 512u + (t & 31u) * 16u + ((t & 127u) >> 5) * 4u + ((k & 127u) >> 5);
}
__device__ __forceinline__ int q_log2_or_neg(int v) { return (v & (v - 1)) == 0 ? 31 - __clz(v) : -1; }

// ---------------------------------------------------------------------------------------------------------------
// Staged epilogue.  A thread of an epilogue warp holds one row of the accumulator (TMEM lane = row), so a 16-byte store
// per thread touches 32 different rows: 32 cache lines per instruction, and with the bf16 copy, the two quantised copies
// and an auxiliary operand per 32 x 32 chunk the load/store path, not the arithmetic, took 17 000 clocks per 128 x 224
// tile against 4 480 clocks of MMAs.  Here every chunk is turned round through the warp's own staging tiles in shared
// memory (swizzled so that both the row-per-thread and the several-threads-per-row accesses are conflict free): it is
// written row-per-thread, read back with four (bf16) or two (E4M3) threads per row and stored with whole row segments
// per group of threads -- 8 or 16 rows per instruction instead of 32 rows of 16 bytes.  The auxiliary operand comes in
// the same way round.  The block maxima along M come from the staged bf16 tile read column-wise (16 conflict-free loads
// per thread and packed bf16 max) instead of 32 `redux.sync` and a selection tree.
// Who stores what was settled by measurement.  With all three copies leaving as TMA stores, their 96 row requests per
// chunk on top of the 240 per K block of the operand loads overran the TMA unit (producer issue time per K block
// 600 -> 790 clocks, 153 us for the c_fc shape); with all three leaving through the load/store unit that pipe was 63 %
// busy over the whole kernel and the epilogue took 10 000 clocks a tile (170 us).  So: a bf16 copy on its own leaves
// through the load/store unit (102 us against 108); when quantised copies are written as well, the bf16 tile leaves as
// one TMA store and the E4M3 tiles through the load/store unit.
// ---------------------------------------------------------------------------------------------------------------
// TMA store of a staged 32 x 32 bf16 tile (the bf16 copy when quantised copies are written too: see below)
__device__ __forceinline__ void q_tma_store_3d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void q_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void q_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void q_sts8(uint32_t a, uint32_t v) { asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void q_sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ uint4 q_lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t q_lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void q_sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t q_max_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// One epilogue warp's chunks of a tile: `stg` / `scratch` are the warp's staging tiles and scratch floats.
template <int EPI, bool WQ, bool WT>
__device__ __forceinline__ void q_staged_tile(const Mx2Params& p, const CUtensorMap* tm_d, uint32_t taddr0, uint32_t stg, uint32_t scratch, int b, int row0, int ncol0, int lane, int sub,
                                              int nchunks QEPI_ARG) {       // `sub`: the warp's first chunk of this tile (rotates from tile to tile)
  constexpr bool kNeedR = EPI == GE_BF16_RES || EPI == GE_MUL_2SQRT;
  constexpr bool kDTma = WQ || WT;                          // the bf16 copy leaves as a TMA store
  if (row0 >= p.M) return;                                  // warp-uniform: the whole warp lies beyond M
  const int row = row0 + lane;
  const bool row_ok = row < p.M;
  const bool ragged = row0 + 32 > p.M;                      // warp-uniform: some of the warp's rows lie beyond M
  const uint32_t sw64 = (uint32_t)((lane >> 1) & 3), sw32 = (uint32_t)((lane >> 2) & 1);
  const uint32_t d_row = stg + QSTG_D + (uint32_t)lane * 64u;
  const uint32_t q_row = stg + QSTG_Q + (uint32_t)lane * 32u;
  const uint32_t t_row = stg + QSTG_T + (uint32_t)lane * 32u;
  const int r_sub = lane >> 2, r_piece = lane & 3;          // coalesced loads of the auxiliary operand: four threads per row
  const __nv_bfloat16* Rb = reinterpret_cast<const __nv_bfloat16*>(p.R) + (long long)b * p.strideR;
  __nv_bfloat16* Dbase = p.D ? reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)b * p.strideD : nullptr;
  const uint32_t kblocks_n = (uint32_t)((p.N + 127) >> 7), kblocks_m = (uint32_t)((p.M + 127) >> 7);
  const int qshift = q_log2_or_neg(p.dq_group), tshift = q_log2_or_neg(p.dt_group);
  uint8_t* sfq = WQ ? p.Dsf + (size_t)b * p.dsf_batch + q_sf_offset32((uint32_t)row, 0u, kblocks_n, p.dq_group, qshift) : nullptr;
  const uint32_t sfq_step = (((uint32_t)p.dq_group + 127u) >> 7) * 512u;          // per 128 columns
  uint8_t* sft = WT ? p.Dtsf + (size_t)b * p.dtsf_batch : nullptr;
  // staged bf16 tile, four threads per row: the address of this thread's piece in rows r_sub + 8 i
  uint32_t t_in[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t rr = (uint32_t)(i * 8 + r_sub);
    t_in[i] = stg + QSTG_D + rr * 64u + ((((uint32_t)r_piece) ^ ((rr >> 1) & 3u)) << 4);
  }
#pragma unroll 1
  for (int c = sub; c < nchunks; c += kEpiWarpsQ / 4) {
    const int col0 = ncol0 + c * 32;
    if (col0 >= p.N) break;                        // warp-uniform: the ragged last tile's columns beyond N
    QEPI_ADD(4);
    if (kDTma) {
      if (elect_one()) q_bulk_wait_read();         // the store of the warp's previous bf16 tile has read the staging tile
    }
    QEPI_ADD(1);
    uint4 rin[4];
    if (kNeedR) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rr = row0 + i * 8 + r_sub, cc = col0 + r_piece * 8;
        rin[i] = make_uint4(0u, 0u, 0u, 0u);
        if (rr < p.M && cc < p.N) rin[i] = *reinterpret_cast<const uint4*>(Rb + (long long)rr * p.ldr + cc);
      }
    }
    uint32_t r[32];
    __syncwarp();
    QEPI_ADD(2);
    BONES_TMEM_LD32(taddr0 + (uint32_t)(c * 32), r);
    tmem_ld_wait();
    QEPI_ADD(0);
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (ragged) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = row_ok ? v[j] : 0.f;
    }
    if (p.alpha != 1.0f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
    }
    if (kNeedR) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t rr = (uint32_t)(i * 8 + r_sub);
        q_sts128(stg + QSTG_D + rr * 64u + ((((uint32_t)r_piece) ^ ((rr >> 1) & 3u)) << 4), rin[i].x, rin[i].y, rin[i].z, rin[i].w);
      }
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 u = q_lds128(d_row + ((((uint32_t)j) ^ sw64) << 4));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float2 f = unpack_bf16(w[t]);
          if (EPI == GE_BF16_RES) {
            v[j * 8 + 2 * t] = fmaf(p.beta, f.x, v[j * 8 + 2 * t]);
            v[j * 8 + 2 * t + 1] = fmaf(p.beta, f.y, v[j * 8 + 2 * t + 1]);
          } else {
            v[j * 8 + 2 * t] *= 2.0f * sqrt_fast(f.x);
            v[j * 8 + 2 * t + 1] *= 2.0f * sqrt_fast(f.y);
          }
        }
      }
      __syncwarp();
    } else if (EPI == GE_RELU2) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float t = fmaxf(v[j], 0.0f);
        v[j] = t * t;
      }
    }
    // bf16 tile: the copy that leaves as D and the source of the column maxima
#pragma unroll
    for (int j = 0; j < 4; ++j)
      q_sts128(d_row + ((((uint32_t)j) ^ sw64) << 4), pack_bf16(v[j * 8 + 0], v[j * 8 + 1]), pack_bf16(v[j * 8 + 2], v[j * 8 + 3]),
               pack_bf16(v[j * 8 + 4], v[j * 8 + 5]), pack_bf16(v[j * 8 + 6], v[j * 8 + 7]));
    if (WQ) {                                      // along N: the thread's 32 values are one block
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
      int biased;
      const float inv = q_scale_pow2(amax, biased);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t o[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = hh * 4 + jj;
          o[jj] = q_pack_e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
        }
        q_sts128(q_row + ((((uint32_t)hh) ^ sw32) << 4), o[0], o[1], o[2], o[3]);
      }
      if (row_ok) sfq[(uint32_t)(col0 >> 7) * sfq_step + (uint32_t)((col0 & 127) >> 5)] = (uint8_t)biased;
    }
    QEPI_ADD(2);
    if (WT) {
      __syncwarp();                                // the bf16 tile is complete
      // along M: a block is one column over the warp's 32 rows (rows beyond M were zeroed).  Four threads per row as in
      // the read-back below: thread (r_sub, r_piece) reads the 8 columns of its piece in rows r_sub + 8 i, folds the four
      // rows, and three shuffles fold the eight threads of the piece.
      uint32_t cm[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 u = q_lds128(t_in[i]);
        cm[0] = q_max_bf16x2(cm[0], u.x & 0x7fff7fffu);
        cm[1] = q_max_bf16x2(cm[1], u.y & 0x7fff7fffu);
        cm[2] = q_max_bf16x2(cm[2], u.z & 0x7fff7fffu);
        cm[3] = q_max_bf16x2(cm[3], u.w & 0x7fff7fffu);
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        cm[t] = q_max_bf16x2(cm[t], __shfl_xor_sync(0xffffffffu, cm[t], 4));
        cm[t] = q_max_bf16x2(cm[t], __shfl_xor_sync(0xffffffffu, cm[t], 8));
        cm[t] = q_max_bf16x2(cm[t], __shfl_xor_sync(0xffffffffu, cm[t], 16));
      }
      // thread (r_sub, r_piece) derives the scale of column r_piece * 8 + r_sub
      const uint32_t pair = (r_sub & 4) ? ((r_sub & 2) ? cm[3] : cm[2]) : ((r_sub & 2) ? cm[1] : cm[0]);
      int biased;
      const float my_inv = q_scale_pow2(__uint_as_float((r_sub & 1) ? (pair & 0xffff0000u) : (pair << 16)), biased);
      sft[q_sf_offset32((uint32_t)(col0 + r_piece * 8 + r_sub), (uint32_t)row0, kblocks_m, p.dt_group, tshift)] = (uint8_t)biased;
      q_sts32(scratch + (uint32_t)(r_piece * 8 + r_sub) * 4u, __float_as_uint(my_inv));
      __syncwarp();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {             // 16 columns = one 16-byte piece of the staged row at a time
        uint32_t o[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j4 = hh * 4 + jj;
          const uint4 sc = q_lds128(scratch + (uint32_t)j4 * 16u);      // four columns' inverse scales, the same on every lane
          o[jj] = q_pack_e4m3x4(v[j4 * 4] * __uint_as_float(sc.x), v[j4 * 4 + 1] * __uint_as_float(sc.y), v[j4 * 4 + 2] * __uint_as_float(sc.z),
                                v[j4 * 4 + 3] * __uint_as_float(sc.w));
        }
        q_sts128(t_row + ((((uint32_t)hh) ^ sw32) << 4), o[0], o[1], o[2], o[3]);
      }
    }
    QEPI_ADD(3);
    if (kDTma && Dbase != nullptr) fence_proxy_async_smem();
    __syncwarp();
    // out: whole row segments per group of threads
    if (kDTma) {
      if (Dbase != nullptr && elect_one()) {
        q_tma_store_3d(tm_d, stg + QSTG_D, col0, row0, b);
        q_bulk_commit();
      }
    } else if (Dbase != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t rr = (uint32_t)(i * 8 + r_sub);
        const uint4 u = q_lds128(stg + QSTG_D + rr * 64u + ((((uint32_t)r_piece) ^ ((rr >> 1) & 3u)) << 4));
        const int grow = row0 + (int)rr, cc = col0 + r_piece * 8;
        if (grow < p.M) {
          __nv_bfloat16* dst = Dbase + (long long)grow * p.ldd + cc;
          if (cc + 8 <= p.N) {
            *reinterpret_cast<uint4*>(dst) = u;
          } else if (cc < p.N) {                     // ragged N: the last piece element by element
            const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
            for (int e = 0; e < p.N - cc; ++e) reinterpret_cast<uint16_t*>(dst)[e] = (uint16_t)(w4[e >> 1] >> ((e & 1) * 16));
          }
        }
      }
    }
    if (WQ || WT) {
      const int h_sub = lane >> 1, h_piece = lane & 1;       // two threads per 32-byte row
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t rr = (uint32_t)(i * 16 + h_sub);
        const uint32_t off = rr * 32u + ((((uint32_t)h_piece) ^ ((rr >> 2) & 1u)) << 4);
        const long long g = ((long long)b * p.M + row0 + (int)rr) * p.N + col0 + h_piece * 16;
        if (row0 + (int)rr < p.M) {
          if (WQ) *reinterpret_cast<uint4*>(p.Dq + g) = q_lds128(stg + QSTG_Q + off);
          if (WT) *reinterpret_cast<uint4*>(p.Dt + g) = q_lds128(stg + QSTG_T + off);
        }
      }
    }
  }
}


// kVariant: which quantised copies the epilogue writes (bit 0 along N, bit 1 along M).  One kernel per variant: with all
// sixteen (epilogue, variant) bodies inlined behind one switch the register allocator spilled inside the chunk loop.
template <int kEpiWarps, int kVariant>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(96 + 32 * kEpiWarps, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const __grid_constant__ CUtensorMap tma_sfa, const __grid_constant__ CUtensorMap tma_sfb,
                       const __grid_constant__ CUtensorMap tma_d, const Mx2Params p) {
  static_assert(kEpiWarps == kEpiWarpsQ, "the staging tiles are laid out for twelve epilogue warps");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t bars = base + QBARS_BASE;
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (QSTAGES + s); };
  auto tfull = [&](int a) { return bars + 8u * (2 * QSTAGES + a); };
  auto tempty = [&](int a) { return bars + 8u * (2 * QSTAGES + 2 + a); };
  auto sffull = [&](int i) { return bars + 8u * (2 * QSTAGES + 4 + i); };
  auto sfempty = [&](int i) { return bars + 8u * (2 * QSTAGES + 4 + kSfSetsMax + i); };
  const uint32_t tmem_slot = bars + 8u * kNumBars;
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + QBARS_BASE + 8 * kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + QBARS_BASE + 8 * kNumBars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = q_cluster_ctarank();
  const bool leader = rank == 0;
  const int bn = p.bn, half_n = p.bn >> 1;
  const int nstages = p.staged ? QSTAGES_STAGED : QSTAGES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < QSTAGES; ++s) {
      mbar_init(full(s), 2);        // leader: its own arrive.expect_tx + the peer's remote arrive
      mbar_init(empty(s), 1);       // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull(a), 1);       // one multicast commit
      mbar_init(tempty(a), 2 * kEpiWarps);     // leader: the epilogue warps of both CTAs
    }
    for (int i = 0; i < kSfSetsMax; ++i) {
      mbar_init(sffull(i), 1);      // the scale-copy thread's commit
      mbar_init(sfempty(i), 1);     // the MMA thread's commit
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
    tma_prefetch_desc(&tma_sfa);
    tma_prefetch_desc(&tma_sfb);
  }
  q_cluster_sync();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  q_cluster_sync();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_g;

  const int base_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int total = base_tiles * p.splits;
  const int KB = p.K / QK;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
  // bytes each CTA brings per stage (the leader's barrier expects both CTAs' bytes)
  const uint32_t b_bytes = p.b_major ? QB_BYTES : (uint32_t)half_n * QK;
  const uint32_t cta_bytes = QA_BYTES + b_bytes + QSFA_BYTES + QSFB_BYTES;

  // The three issuing roles run on all 32 lanes of their warp with warp-uniform state and issue from the elected lane
  // (see `elect_one`).  A lane whose bounded wait ran out turns `dead`: it keeps walking the loops without waiting or
  // issuing, so the warp stays together for the `elect.sync` of every iteration and reaches the tear-down as one.
  if (warp == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool dead = false;
    QPROF_DECL(2);
    for (int tile = cluster_id; tile < total; tile += n_clusters) {
      int b, mb, nb;
      const int sp = p.splits == 1 ? 0 : tile / base_tiles;
      decode_tile_q(tile - sp * base_tiles, p.tiles_m, p.tiles_n, b, mb, nb);
      const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
      const int m0 = mb * QM + (int)rank * 128, n0 = nb * bn + (int)rank * half_n;
      const int sfa_row = b * p.sfa_rows_per_batch + (2 * mb + (int)rank) * KB * 2;      // 256-byte rows, 2 per chunk
      const int sfb_row = b * p.sfb_rows_per_batch + nb * KB * 4;                         // 4 per (tile, K block)
      for (int kb = kb0; kb < kb1; ++kb) {
        QPROF_ADD(1);
        if (!dead) dead = !mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.err, ERR_WAIT_EMPTY);
        QPROF_ADD(0);
        const uint32_t sa = base + stage * QSTAGE_STRIDE, sb = sa + QA_BYTES, ssfa = sb + QB_BYTES, ssfb = ssfa + QSFA_BYTES;
        if (elect_one() && !dead) {
          if (leader) mbar_arrive_expect_tx(full(stage), 2 * cta_bytes);
          if (p.a_major == 0) q_tma_3d(sa, &tma_a, full(stage), kb * QK, m0, b);
          else                q_tma_3d(sa, &tma_a, full(stage), m0, kb * QK, b);
          if (p.b_major == 0) q_tma_3d(sb, &tma_b, full(stage), kb * QK, n0, b);
          else                q_tma_3d(sb, &tma_b, full(stage), n0, kb * QK, b);
          q_tma_2d(ssfa, &tma_sfa, full(stage), 0, sfa_row + kb * 2);
          q_tma_2d(ssfb, &tma_sfb, full(stage), 0, sfb_row + kb * 4);
          if (!leader) q_mbar_arrive_cluster(full(stage), 0);
        }
        if (++stage == nstages) { stage = 0; phase ^= 1u; }
      }
    }
    QPROF_ADD(1);
    if (lane == 0) { QPROF_STORE(5, 0); QPROF_STORE(6, 1); QPROF_TOTAL(7); }
  } else if (warp == 1) {
    if (leader) {
      // K-major: 32 bytes of K per MMA step (descriptor unit 16 bytes); MN-major: 32 K rows of 128 bytes
      const uint32_t a_step = p.a_major ? (32 * 128) >> 4 : 32 >> 4;
      const uint32_t b_step = p.b_major ? (32 * 128) >> 4 : 32 >> 4;
      const uint32_t a_lbo = p.a_major ? 128 * 128 : 0, b_lbo = p.b_major ? 128 * 128 : 0;
      int stage = 0, acc = 0, sfset = 0;
      uint32_t phase = 0, acc_phase = 0, sf_phase = 0;
      bool dead = false;
      uint32_t idesc[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        idesc[k] = umma_idesc_mxf8(QM, (uint32_t)bn, 0, 0, (uint32_t)p.a_major, (uint32_t)p.b_major, (uint32_t)k, (uint32_t)k);
      // descriptors of stage 0; a stage adds QSTAGE_STRIDE >> 4 to the address field
      const uint64_t adesc0 = umma_smem_desc(base, a_lbo, 1024, kLayoutSw128);
      const uint64_t bdesc0 = umma_smem_desc(base + QA_BYTES, b_lbo, 1024, kLayoutSw128);
      const uint64_t sdesc0 = umma_smem_desc(base + QA_BYTES + QB_BYTES, 0, 128, kLayoutNone);
      QPROF_DECL(9);
      for (int tile = cluster_id; tile < total; tile += n_clusters) {
        QPROF_ADD(3);
        if (!dead) dead = !mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        QPROF_ADD(0);
        QPROF_COUNT(5);
        tc_fence_after();
        const uint32_t d_tmem = tmem + (uint32_t)(acc * bn);
        const int sp = p.splits == 1 ? 0 : tile / base_tiles;
        const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          QPROF_ADD(3);
          // With the scale-copy warp, its commit on `sffull` implies the stage's data: that warp waited for `full[s]`
          // before it copied.  Waiting for `full[s]` here as well cost about 100 clocks per K block.
          if (!p.sf_warp) {
            if (!dead) dead = !mbar_wait(full(stage), phase, abort_flag, p.err, ERR_WAIT_FULL);
          }
          QPROF_ADD(1);
          QPROF_COUNT(4);
          const uint64_t soff = (uint64_t)(stage * (QSTAGE_STRIDE >> 4));
          const uint32_t sfa_t = tmem + QTMEM_SF0 + (uint32_t)sfset * QTMEM_SF_STRIDE, sfb_t = sfa_t + 4;
          if (p.sf_warp) {
            if (!dead) dead = !mbar_wait(sffull(sfset), sf_phase, abort_flag, p.err, ERR_WAIT_AUX);
          }
          QPROF_ADD(2);
          tc_fence_after();
          const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
          QPROF_ADD(3);
          if (elect_one() && !dead) {
            if (!p.sf_warp) {
              q_cp_sf_pair(sfa_t, sdesc0 + soff);
              q_cp_sf_pair(sfb_t, sdesc0 + soff + (QSFA_BYTES >> 4));
              q_cp_sf_pair(sfb_t + 4, sdesc0 + soff + ((QSFA_BYTES + 512) >> 4));
            }
#pragma unroll
            for (int k = 0; k < QK / 32; ++k)
              q_umma_mxf8_pair(d_tmem, adesc + (uint64_t)(k * a_step), bdesc + (uint64_t)(k * b_step), idesc[k], ((kb - kb0) | k) ? 1u : 0u,
                               sfa_t, sfb_t);
            q_commit_pair(empty(stage));
            if (p.sf_warp) q_commit_local(sfempty(sfset));        // this set of scale columns is free once these MMAs are done
            if (kb == kb1 - 1) q_commit_pair(tfull(acc));
          }
          QPROF_ADD(6);
          if (++stage == nstages) { stage = 0; phase ^= 1u; }
          if (++sfset == p.sf_sets) { sfset = 0; sf_phase ^= 1u; }
        }
        if (++acc == p.acc_stages) { acc = 0; acc_phase ^= 1u; }
      }
      QPROF_ADD(3);
      if (lane == 0) {
        QPROF_STORE(0, 0); QPROF_STORE(1, 1); QPROF_STORE(2, 2); QPROF_STORE(3, 3); QPROF_TOTAL(4); QPROF_STORE(14, 4); QPROF_STORE(15, 5);
        QPROF_STORE(16, 6);
      }
    }
  } else if (warp == 2) {
    // Scale-copy warp (leader only): `tcgen05.cp` of a K block's scales into the next free set of scale columns, as
    // soon as the block's data has landed, running up to `sf_sets` blocks ahead of the MMA warp.  Issued from the MMA
    // warp itself the copies sit in its in-order stream between two blocks' MMAs, and the tensor pipe was measured at
    // 42-55 % active; from a warp of their own they can complete while the previous block's MMAs execute.
    if (leader && p.sf_warp) {
      int stage = 0, sfset = 0;
      uint32_t phase = 0, sf_phase = 0;
      bool dead = false;
      const uint64_t sdesc0 = umma_smem_desc(base + QA_BYTES + QB_BYTES, 0, 128, kLayoutNone);
      QPROF_DECL(3);
      for (int tile = cluster_id; tile < total; tile += n_clusters) {
        const int sp = p.splits == 1 ? 0 : tile / base_tiles;
        const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          QPROF_ADD(2);
          if (!dead) dead = !mbar_wait(full(stage), phase, abort_flag, p.err, ERR_WAIT_FULL);
          QPROF_ADD(0);
          if (!dead) dead = !mbar_wait(sfempty(sfset), sf_phase ^ 1u, abort_flag, p.err, ERR_WAIT_AUX);
          QPROF_ADD(1);
          tc_fence_after();
          const uint64_t soff = (uint64_t)(stage * (QSTAGE_STRIDE >> 4));
          const uint32_t sfa_t = tmem + QTMEM_SF0 + (uint32_t)sfset * QTMEM_SF_STRIDE, sfb_t = sfa_t + 4;
          if (elect_one() && !dead) {
            q_cp_sf_pair(sfa_t, sdesc0 + soff);
            q_cp_sf_pair(sfb_t, sdesc0 + soff + (QSFA_BYTES >> 4));
            q_cp_sf_pair(sfb_t + 4, sdesc0 + soff + ((QSFA_BYTES + 512) >> 4));
            q_commit_local(sffull(sfset));
          }
          if (++stage == nstages) { stage = 0; phase ^= 1u; }
          if (++sfset == p.sf_sets) { sfset = 0; sf_phase ^= 1u; }
        }
      }
      QPROF_ADD(2);
      if (lane == 0) { QPROF_STORE(8, 0); QPROF_STORE(9, 1); QPROF_STORE(10, 2); }
    }
  } else {
    // epilogue warps: kEpiWarps / 4 per 32-lane TMEM quadrant (a warp reaches the quadrant warp % 4); the warps of a
    // quadrant take every (kEpiWarps / 4)-th 32-column chunk
    const int q = warp & 3, sub = (warp - 3) >> 2;
    const int nchunks = bn >> 5;
    const bool f32out = p.epi == GE_ACC_F32;
    const uint32_t stg = base + QSTG_BASE + (uint32_t)(warp - 3) * QSTG_BYTES;
    const uint32_t scratch = base + QSCRATCH_BASE + (uint32_t)(warp - 3) * QSTG_SCRATCH;
    int acc = 0, tile_iter = 0;
    uint32_t acc_phase = 0;
    QPROF_DECL(2);
#ifdef BONES_MX_PROF
    long long qe_[5] = {};
    long long qe_t_ = clock64();
#endif
    for (int tile = cluster_id; tile < total; tile += n_clusters) {
      int b, mb, nb;
      decode_tile_q(tile % base_tiles, p.tiles_m, p.tiles_n, b, mb, nb);
      const int row0 = mb * QM + (int)rank * 128 + q * 32;
      QPROF_ADD(1);
      const bool got = mbar_wait(tfull(acc), acc_phase, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      QPROF_ADD(0);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const uint32_t taddr0 = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * bn);
      // the three warps of a quadrant take every third chunk; which of them starts at chunk 0 rotates from tile to tile,
      // so with seven or eight chunks a tile the odd one falls on each warp in turn
      const int first = (sub + tile_iter) % (kEpiWarps / 4);
      ++tile_iter;
      if (!p.staged) {
        // fp32 accumulate (split-K weight gradients) or a bf16 result whose pitch does not allow a TMA store
        const int row = row0 + lane;
        const bool row_ok = row < p.M;
        const long long drow = (long long)b * p.strideD + (long long)row * p.ldd;
        const long long rrow = (long long)b * p.strideR + (long long)row * p.ldr;
#pragma unroll 1
        for (int c = first; c < nchunks; c += kEpiWarps / 4) {
          uint32_t r[32];
          __syncwarp();
          BONES_TMEM_LD32(taddr0 + (uint32_t)(c * 32), r);
          tmem_ld_wait();
          const int col0 = nb * bn + c * 32;
          if (col0 >= p.N || !row_ok) continue;
          const size_t esz = f32out ? 4 : 2;
          uint4 nopre[4];
          gemm_store_chunk(r, p.epi, p.alpha, p.beta, p.wide != 0, p.splits > 1 || p.atomic, reinterpret_cast<uint8_t*>(p.D) + (drow + col0) * esz,
                           reinterpret_cast<const uint8_t*>(p.R) + (rrow + col0) * esz, false, nopre, min(32, p.N - col0));
        }
      } else {
#ifdef BONES_MX_PROF
        qe_t_ = clock64();
#endif
#define BONES_Q_TILE(E, WQ, WT) q_staged_tile<E, WQ, WT>(p, &tma_d, taddr0, stg, scratch, b, row0, nb * bn, lane, first, nchunks QEPI_PASS)
#define BONES_Q_EPI(WQ, WT)                                         \
  switch (p.epi) {                                                  \
    case GE_BF16_RES: BONES_Q_TILE(GE_BF16_RES, WQ, WT); break;     \
    case GE_RELU2: BONES_Q_TILE(GE_RELU2, WQ, WT); break;           \
    case GE_MUL_2SQRT: BONES_Q_TILE(GE_MUL_2SQRT, WQ, WT); break;   \
    default: BONES_Q_TILE(GE_BF16, WQ, WT); break;                  \
  }
        BONES_Q_EPI((kVariant & 1) != 0, (kVariant & 2) != 0)
#undef BONES_Q_EPI
#undef BONES_Q_TILE
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) q_mbar_arrive_cluster(tempty(acc), 0);
      if (++acc == p.acc_stages) { acc = 0; acc_phase ^= 1u; }
    }
    __syncwarp();
    if (p.staged && elect_one()) q_bulk_wait_read();          // the last TMA store has read its staging tile
    QPROF_ADD(1);
    if (warp == 3 && lane == 0) {
      QPROF_STORE(11, 0); QPROF_STORE(12, 1); QPROF_TOTAL(13);
#ifdef BONES_MX_PROF
      if (p.prof) for (int i = 0; i < 5; ++i) p.prof[(long long)blockIdx.x * 32 + 19 + i] = qe_[i];
#endif
    }
  }

  // tear-down: both CTAs of the pair always arrive here (every wait above is bounded)
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  q_cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Quantiser for both axes in one pass: x bf16 [R, C] -> q_row (blocks of 32 along C) and q_col (blocks of 32 along R),
// each with its scale chunks.  Persistent: one CTA per SM, twelve warps, each warp a pipeline of its own.  A warp tile is
// 32 rows x 128 columns (one K block of the row copy, so a row's four scale bytes leave as one 32-bit store); its 32
// rows of 256 bytes arrive as bulk asynchronous copies (one per lane) in one of the warp's two 8 KB stages, signalled
// by an mbarrier.  The warp copies a landed tile into registers, hands the stage straight back to the copy engine for
// the tile after next, and then does the arithmetic, so that about two tiles per warp (190 KB per SM) are in flight
// whatever the arithmetic is doing.  (With plain loads the kernel waited on them: 13 instructions per value, 35 % of
// the issue slots, 47 % of the DRAM bandwidth, nearly all stalls on the loads' scoreboard.)
// Eight threads per row: thread (rsub = lane / 8, piece = lane % 8) holds the 8 values of columns piece * 8 .. + 7 of
// each 64-column half in rows rsub, rsub + 4, ..., rsub + 28.  A quarter warp reads 128 contiguous bytes of shared
// memory (conflict free) and stores 64 contiguous bytes per row; a row block's maximum needs two shuffles among the
// four threads of the block and a column block's maximum two among the four threads of the column group.
// All 32 rows (and the 32 columns of a chunk) fall into one scale tile because the tile heights are multiples of 32,
// so the scale offsets are a base plus a lane term: no per-row division and no 64-bit index arithmetic.  Values are
// scaled as packed bf16 pairs (a power of two: exact) before the conversion.
// ---------------------------------------------------------------------------------------------------------------
constexpr int QD_STAGES = 2;
// kHalves 64-column halves per warp tile (2: a whole K block of the row copy per tile; 1: half of one, which needs fewer
// registers and half the shared memory per warp, so more warps fit an SM), kWarps warps per CTA
template <int kHalves, int kWarps>
struct QdGeom {
  static constexpr int kTileBytes = 32 * 128 * kHalves;
  static constexpr int kBarsBase = kWarps * QD_STAGES * kTileBytes;
  static constexpr int kSmemBytes = kBarsBase + kWarps * QD_STAGES * 8 + 16;
};
__device__ __forceinline__ uint32_t q_mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// From the bf16 bit pattern of a block's largest magnitude: the biased UE8M0 exponent of the smallest power of two 2^e with
// amax / 2^e <= 448, and 2^-e as a bf16 pair (the same rule as q_scale_pow2; an all-zero block gets exponent 0).
__device__ __forceinline__ uint32_t q_scale_bf16(uint32_t amax16, uint32_t& biased) {
  const int b = max((int)(amax16 >> 7) - 8 + ((amax16 & 0x7fu) > 0x60u ? 1 : 0), 0);
  biased = (uint32_t)b;
  return ((uint32_t)(254 - b) << 7) * 0x10001u;
}
// 8 bf16 values (4 packed words) times their packed power-of-two factors -> 8 E4M3 bytes
__device__ __forceinline__ uint2 q_cvt_e4m3x8(const uint32_t (&w)[4], const uint32_t (&inv2)[4]) {
  uint32_t s[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) s[t] = q_mul_bf16x2(w[t], inv2[t]);
  return make_uint2(q_pack_e4m3x4(__uint_as_float(s[0] << 16), __uint_as_float(s[0] & 0xffff0000u), __uint_as_float(s[1] << 16),
                                  __uint_as_float(s[1] & 0xffff0000u)),
                    q_pack_e4m3x4(__uint_as_float(s[2] << 16), __uint_as_float(s[2] & 0xffff0000u), __uint_as_float(s[3] << 16),
                                  __uint_as_float(s[3] & 0xffff0000u)));
}
// part of a scale offset shared by rows r0 .. r0 + 31 of one scale tile (r0 and the tile height multiples of 32) at
// K block `kb`; a row r0 + j adds j * 16 and the 32-wide block `ks` of the K block adds ks
__device__ __forceinline__ size_t q_sf_base32(uint32_t r0, uint32_t kb, uint32_t kblocks, int group) {
  const uint32_t g = r0 / (uint32_t)group;
  const uint32_t t0 = r0 - g * (uint32_t)group;
  const uint32_t chunks = ((uint32_t)group + 127u) >> 7;
  return ((size_t)g * kblocks + kb) * (size_t)(chunks * 512u) + (size_t)((t0 >> 7) * 512u + ((t0 & 127u) >> 5) * 4u);
}
template <bool kRow, bool kCol, int kHalves, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, 1)
mx_quant_dual_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ qr, uint8_t* __restrict__ sfr, int group_r,
                     uint8_t* __restrict__ qc, uint8_t* __restrict__ sfc, int group_c, long long R, long long C, uint32_t n_tiles, int* err) {
  using G = QdGeom<kHalves, kWarps>;
  constexpr int kCols = 64 * kHalves, kPitch = 2 * kCols;        // columns of a tile; bytes of a tile row in shared memory
  extern __shared__ __align__(128) uint8_t qd_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, rsub = lane >> 3, piece = lane & 7;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(qd_smem + G::kBarsBase + kWarps * QD_STAGES * 8);
  const uint32_t stage0 = smem_u32(qd_smem) + (uint32_t)(warp * QD_STAGES * G::kTileBytes);
  const uint32_t bar0 = smem_u32(qd_smem) + (uint32_t)(G::kBarsBase + warp * QD_STAGES * 8);
  if (threadIdx.x == 0) *abort_flag = 0;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < QD_STAGES; ++s) mbar_init(bar0 + 8u * s, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const uint32_t tiles_c = (uint32_t)(C / kCols);
  const uint32_t stride = gridDim.x * kWarps;
  const uint32_t kb_c = (uint32_t)((C + 127) >> 7), kb_r = (uint32_t)((R + 127) >> 7);
  // the rows of tile `tile` into stage s: every lane copies one row
  auto issue = [&](uint32_t tile, int s) {
    const uint32_t tr = tile / tiles_c, tc = tile - tr * tiles_c;
    const long long row0 = (long long)tr * 32;
    const int rows_here = (int)min((long long)32, R - row0);
    if (lane == 0) mbar_arrive_expect_tx(bar0 + 8u * s, (uint32_t)(rows_here * kPitch));
    __syncwarp();
    if (lane < rows_here)
      bulk_load(stage0 + (uint32_t)(s * G::kTileBytes + lane * kPitch), x + (row0 + lane) * ldx + (long long)tc * kCols, (uint32_t)kPitch,
                bar0 + 8u * s);
  };
  const uint32_t first = blockIdx.x * kWarps + warp;
#pragma unroll
  for (int s = 0; s < QD_STAGES; ++s)
    if (first + s * stride < n_tiles) issue(first + s * stride, s);
  int n = 0;
  for (uint32_t tile = first; tile < n_tiles; tile += stride, ++n) {
    const int s = n & 1;
    const bool got = mbar_wait(bar0 + 8u * s, (uint32_t)((n >> 1) & 1), abort_flag, err, ERR_WAIT_FULL);
    if (!__all_sync(0xffffffffu, got)) break;
    const uint32_t tr = tile / tiles_c, tc = tile - tr * tiles_c;
    const long long row0 = (long long)tr * 32;
    const int rows_here = (int)min((long long)32, R - row0);
    // the tile's place in its 128-column K block of the row copy: first chunk and K block
    const uint32_t kblock = kHalves == 2 ? tc : (tc >> 1);
    const int chunk0 = kHalves == 2 ? 0 : (int)(tc & 1u) * 2;
    uint4 raw[kHalves][8];
    {
      const uint8_t* st = qd_smem + (warp * QD_STAGES + s) * G::kTileBytes + rsub * kPitch + piece * 16;
#pragma unroll
      for (int h = 0; h < kHalves; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i)
          raw[h][i] = i * 4 + rsub < rows_here ? *reinterpret_cast<const uint4*>(st + i * 4 * kPitch + h * 128) : make_uint4(0u, 0u, 0u, 0u);
    }
    // the stage goes back to the copy engine for the tile after next
    fence_proxy_async_smem();
    __syncwarp();
    if (tile + 2 * stride < n_tiles) issue(tile + 2 * stride, s);

    const long long q0 = (row0 + rsub) * C + (long long)tc * kCols + piece * 8;   // this thread's first output byte, either copy
    const long long qstep = 4 * C;
    uint32_t rowsf[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};      // scale bytes of the row's blocks that this thread saw
#pragma unroll
    for (int h = 0; h < kHalves; ++h) {
      const int c = 2 * h + (piece >> 2);                        // this thread's 32-column chunk within the tile
      uint32_t cm[4] = {0u, 0u, 0u, 0u};                         // packed bf16 maxima of this thread's 8 columns over its 8 rows
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t w[4] = {raw[h][i].x, raw[h][i].y, raw[h][i].z, raw[h][i].w};
        uint32_t a[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          a[t] = w[t] & 0x7fff7fffu;
          if (kCol) cm[t] = q_max_bf16x2(cm[t], a[t]);
        }
        if (kRow) {
          uint32_t m2 = q_max_bf16x2(q_max_bf16x2(a[0], a[1]), q_max_bf16x2(a[2], a[3]));
          m2 = q_max_bf16x2(m2, __shfl_xor_sync(0xffffffffu, m2, 1));
          m2 = q_max_bf16x2(m2, __shfl_xor_sync(0xffffffffu, m2, 2));
          uint32_t biased;
          const uint32_t inv = q_scale_bf16(max(m2 & 0xffffu, m2 >> 16), biased);
          const uint32_t inv2[4] = {inv, inv, inv, inv};
          const uint2 o = q_cvt_e4m3x8(w, inv2);
          if (i * 4 + rsub < rows_here) *reinterpret_cast<uint2*>(qr + q0 + i * qstep + h * 64) = o;
          rowsf[i] |= biased << (8 * c);
        }
      }
      if (kCol) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          cm[t] = q_max_bf16x2(cm[t], __shfl_xor_sync(0xffffffffu, cm[t], 8));
          cm[t] = q_max_bf16x2(cm[t], __shfl_xor_sync(0xffffffffu, cm[t], 16));
        }
        // thread (rsub, piece) derives the scales of columns piece * 8 + 2 rsub and + 1 of the half (word rsub of its four)
        const uint32_t pair = (rsub & 2) ? ((rsub & 1) ? cm[3] : cm[2]) : ((rsub & 1) ? cm[1] : cm[0]);
        uint32_t b_lo, b_hi;
        const uint32_t inv_lo = q_scale_bf16(pair & 0xffffu, b_lo), inv_hi = q_scale_bf16(pair >> 16, b_hi);
        const uint32_t my_inv2 = (inv_lo & 0xffffu) | (inv_hi & 0xffff0000u);
        // the transposed operand's "rows" are the columns; its K block is the 128-row block of row0
        uint8_t* sp = sfc + q_sf_base32(tc * (uint32_t)kCols + (uint32_t)c * 32u, (uint32_t)(row0 >> 7), kb_r, group_c) +
                      (size_t)(((piece & 3) * 8 + 2 * rsub) * 16 + (int)((row0 & 127) >> 5));
        sp[0] = (uint8_t)b_lo;
        sp[16] = (uint8_t)b_hi;
        uint32_t inv2[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) inv2[t] = __shfl_sync(0xffffffffu, my_inv2, (t << 3) | piece);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t w[4] = {raw[h][i].x, raw[h][i].y, raw[h][i].z, raw[h][i].w};
          const uint2 o = q_cvt_e4m3x8(w, inv2);
          if (i * 4 + rsub < rows_here) *reinterpret_cast<uint2*>(qc + q0 + i * qstep + h * 64) = o;
        }
      }
    }
    if (kRow) {
      // pieces 0 and 4 of a row hold the scale bytes of the tile's even and odd chunks; a whole K block's four bytes
      // leave as one 32-bit store, half a block's two as one 16-bit store
      uint8_t* rp = sfr + q_sf_base32((uint32_t)row0, kblock, kb_c, group_r) + (size_t)(rsub * 16 + chunk0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t v = rowsf[i] | __shfl_xor_sync(0xffffffffu, rowsf[i], 4);
        if (piece == 0 && i * 4 + rsub < rows_here) {
          if (kHalves == 2) *reinterpret_cast<uint32_t*>(rp + i * 64) = v;
          else *reinterpret_cast<uint16_t*>(rp + i * 64) = (uint16_t)v;
        }
      }
    }
  }
  // a warp that gave up may still have a copy on its way into shared memory: stay a moment before the CTA's memory goes
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

static int tmap_operand_q(CUtensorMap* out, const void* ptr, int major, long long rows, long long K, long long ld, long long stride, int batch,
                          int box_rows) {
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  if (major == 0) {
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)rows;
    box[0] = QK; box[1] = (uint32_t)box_rows;
  } else {
    dims[0] = (uint64_t)rows; dims[1] = (uint64_t)K;
    box[0] = 128; box[1] = QK;
  }
  dims[2] = (uint64_t)batch;
  box[2] = 1;
  strides[0] = (uint64_t)ld;
  strides[1] = batch > 1 ? (uint64_t)stride : strides[0] * dims[1];
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// bf16 result [batch, M, N], row pitch `ld` and batch pitch `stride` in elements, stored in boxes of 32 x 32 from the
// epilogue's staging tiles (rows of 64 bytes, 64-byte swizzle)
static int tmap_out_q(CUtensorMap* out, const void* ptr, long long M, long long N, long long ld, long long stride, int batch) {
  uint64_t dims[3] = {(uint64_t)N, (uint64_t)M, (uint64_t)batch};
  uint64_t strides[2] = {(uint64_t)(ld * 2), (uint64_t)((batch > 1 ? stride : ld * M) * 2)};
  uint32_t box[3] = {32, 32, 1};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

// scale chunks seen as rows of 256 bytes; a box of `box_rows` rows is one K block's scales of one tile
static int tmap_scales_q(CUtensorMap* out, const void* ptr, long long bytes, int box_rows) {
  uint64_t dims[2] = {256, (uint64_t)(bytes / 256)};
  uint64_t strides[1] = {256};
  uint32_t box[2] = {256, (uint32_t)box_rows};
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace bones

#ifdef BONES_MX_PROF
static long long* g_mx_prof = nullptr;
// measuring build: device buffer of 32 counters per CTA that the next launches fill (null switches it off)
extern "C" void bones_mx2_set_prof(void* buf) { g_mx_prof = (long long*)buf; }
#endif

extern "C" {
using namespace bones;

// Bytes of the scale chunks of one operand: `rows` rows in tiles of `group` rows, contraction length K.
long long bones_mx2_sf_bytes(long long rows, long long K, int group) {
  return ((rows + group - 1) / group) * ((K + 127) >> 7) * ((group + 127) >> 7) * 512;
}

// x bf16 [R, C] -> optional row-quantised copy (qr, sfr: blocks along C, scale tiles of `group_r` rows) and optional
// column-quantised copy (qc, sfc: blocks along R; its scale chunks describe an operand with rows = C, K = R, tiles of
// `group_c` rows).  C a multiple of 128; a last, partial block of rows is quantised as a block of its own.
int bones_mx2_quant(const void* x, long long ldx, void* qr, void* sfr, int group_r, void* qc, void* sfc, int group_c, long long R, long long C,
                    void* stream) {
  if ((C % 128) || (ldx % 8) || ((uintptr_t)x & 15)) return -2;
  if ((qr && ((group_r % 32) || ((uintptr_t)sfr & 3))) || (qc && (group_c % 32)) || R >= (1LL << 31) || C >= (1LL << 31)) return -2;
  if (R == 0 || (!qr && !qc)) return 0;
  // a K block of the row copy per warp tile, twelve warps per SM.  Tiles of half a K block with sixteen or twenty warps
  // (kHalves = 1) were measured slower (0.62 - 0.63 of the copy rate against 0.70 at 131072 x 1280)
  constexpr int kHalves = 2, kWarps = 12;
  const long long tiles = ((R + 31) / 32) * (C / (64 * kHalves));
  if (tiles >= (1LL << 30)) return -2;
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const unsigned grid = (unsigned)std::min<long long>(sms, (tiles + kWarps - 1) / kWarps);
  int* err = error_word();
  using G = QdGeom<kHalves, kWarps>;
  static bool attr_set = false;
  if (!attr_set) {
    BONES_CHECK(cudaFuncSetAttribute(mx_quant_dual_kernel<true, true, kHalves, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes));
    BONES_CHECK(cudaFuncSetAttribute(mx_quant_dual_kernel<true, false, kHalves, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes));
    BONES_CHECK(cudaFuncSetAttribute(mx_quant_dual_kernel<false, true, kHalves, kWarps>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes));
    attr_set = true;
  }
#define BONES_QUANT_LAUNCH(ROW, COL)                                                                                          \
  mx_quant_dual_kernel<ROW, COL, kHalves, kWarps><<<grid, kWarps * 32, G::kSmemBytes, (cudaStream_t)stream>>>(                 \
      (const __nv_bfloat16*)x, ldx, (uint8_t*)qr, (uint8_t*)sfr, group_r, (uint8_t*)qc, (uint8_t*)sfc, group_c, R, C, (uint32_t)tiles, err)
  if (qr && qc) BONES_QUANT_LAUNCH(true, true);
  else if (qr) BONES_QUANT_LAUNCH(true, false);
  else if (qc) BONES_QUANT_LAUNCH(false, true);
#undef BONES_QUANT_LAUNCH
  return (int)cudaGetLastError();
}

// A_q: [batch, M, K] (a_major 0, lda = row pitch in bytes) or [batch, K, M] (a_major 1); likewise B_q with N.  sfa: scale
// chunks with tiles of 128 rows; sfb: with tiles of `bn` rows.  D: bf16 [batch, M, N] (fp32 with epi 3; null when only
// quantised outputs are wanted).  Dq / Dsf: the result quantised along N (scale tiles of `dq_group` rows, K = N);
// Dt / Dtsf: quantised along M (scale chunks of an operand with rows = N in tiles of `dt_group`, K = M).
int bones_gemm_mxfp8_pair(const void* Aq, const void* sfa, const void* Bq, const void* sfb, void* D, const void* R, void* Dq, void* Dsf,
                          int dq_group, void* Dt, void* Dtsf, int dt_group, int M, int N, int K, int batch, long long lda, long long ldb,
                          long long ldd, long long ldr, long long strideA, long long strideB, long long strideD, long long strideR, int a_major,
                          int b_major, int epi, float alpha, float beta, int bn, int splits, int atomic, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((K % 128) || (lda % 16) || (ldb % 16) || ((uintptr_t)Aq & 15) || ((uintptr_t)Bq & 15) || ((uintptr_t)sfa & 15) || ((uintptr_t)sfb & 15))
    return -2;
  if (bn != 160 && bn != 224 && bn != 256) return -3;
  if (b_major && bn != 256) return -4;          // an MN-major B tile is one 128-byte swizzle atom per CTA
  const bool f32out = epi == GE_ACC_F32;
  if (!(epi == GE_BF16 || epi == GE_BF16_RES || epi == GE_RELU2 || epi == GE_ACC_F32 || epi == GE_MUL_2SQRT)) return -5;
  if ((Dq || Dt) && (f32out || (N % 32) || ((Dq != nullptr) && (N % 128)) || ((Dt != nullptr) && (M % 32)))) return -6;
  if (D && (ldd % (f32out ? 4 : 8))) return -7;
  if (!D && !Dq && !Dt) return -8;
  Mx2Params p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_major = a_major; p.b_major = b_major;
  p.bn = bn;
  p.acc_stages = (2 * bn <= (int)QTMEM_SF0) ? 2 : 1;
  {
    static int sets = -1;
    if (sets < 0) {
      const char* e = getenv("BONES_MX_SF_SETS");
      sets = e ? atoi(e) : 4;
      if (sets != 1 && sets != 2 && sets != 4) sets = 4;
    }
    p.sf_sets = sets;
    static int sfw = -1;
    if (sfw < 0) {
      const char* e = getenv("BONES_MX_SF_WARP");
      sfw = e ? (atoi(e) != 0) : 1;
    }
    p.sf_warp = sfw;
  }
  p.epi = epi; p.alpha = alpha; p.beta = beta;
  p.D = D; p.ldd = ldd; p.strideD = strideD;
  p.R = R ? R : D; p.ldr = R ? ldr : ldd; p.strideR = R ? strideR : strideD;
  p.Dq = (uint8_t*)Dq; p.Dsf = (uint8_t*)Dsf; p.dq_group = dq_group > 0 ? dq_group : 128;
  p.Dt = (uint8_t*)Dt; p.Dtsf = (uint8_t*)Dtsf; p.dt_group = dt_group > 0 ? dt_group : 128;
  p.dsf_batch = bones_mx2_sf_bytes(M, N, p.dq_group);
  p.dtsf_batch = bones_mx2_sf_bytes(N, M, p.dt_group);
  p.err = error_word();
#ifdef BONES_MX_PROF
  p.prof = g_mx_prof;
#else
  p.prof = nullptr;
#endif
  const long long wal = f32out ? 8 : 16;
  p.wide = (D && (ldd % wal == 0) && (strideD % wal == 0) && (!R || (ldr % wal == 0 && strideR % wal == 0)) && (((uintptr_t)D & 31) == 0) &&
            (!R || ((uintptr_t)R & 31) == 0)) ? 1 : 0;
  p.tiles_m = (M + QM - 1) / QM;
  p.tiles_n = (N + bn - 1) / bn;
  const int KB = K / QK;
  const long long sfa_bytes = bones_mx2_sf_bytes(M, K, 128), sfb_bytes = bones_mx2_sf_bytes(N, K, bn);
  p.sfa_rows_per_batch = (int)(sfa_bytes / 256);
  p.sfb_rows_per_batch = (int)(sfb_bytes / 256);
  CUtensorMap ta, tb, tsa, tsb;
  int rc = tmap_operand_q(&ta, Aq, a_major, M, K, lda, strideA, batch, 128);
  if (rc) return rc;
  rc = tmap_operand_q(&tb, Bq, b_major, N, K, ldb, strideB, batch, bn / 2);
  if (rc) return rc;
  rc = tmap_scales_q(&tsa, sfa, sfa_bytes * batch, 2);
  if (rc) return rc;
  rc = tmap_scales_q(&tsb, sfb, sfb_bytes * batch, 4);
  if (rc) return rc;
  // bf16 / E4M3 results are turned round through shared memory when their pitches allow 16-byte accesses
  const bool d_tma = !D || ((ldd % 8 == 0) && (strideD % 8 == 0) && (((uintptr_t)D & 15) == 0));
  const bool r_vec = !R || ((ldr % 8 == 0) && (strideR % 8 == 0) && (((uintptr_t)R & 15) == 0));
  // short contractions and quantised copies: the epilogue is the larger part of a tile and gets the staging tiles (at
  // the price of the sixth stage); long contractions keep six stages and store from registers
  p.staged = (!f32out && d_tma && r_vec && (Dq || Dt || K <= 2560)) ? 1 : 0;
  if (!p.staged && (Dq || Dt)) return -7;
  CUtensorMap td;
  memset(&td, 0, sizeof(td));
  if (p.staged && D && (Dq || Dt)) {
    rc = tmap_out_q(&td, D, M, N, ldd, strideD, batch);
    if (rc) return rc;
  }
  constexpr size_t smem = QSMEM_BYTES;
  static bool attr_set = false;
  if (!attr_set) {
    BONES_CHECK(cudaFuncSetAttribute(gemm_mxfp8_pair_kernel<kEpiWarpsQ, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    BONES_CHECK(cudaFuncSetAttribute(gemm_mxfp8_pair_kernel<kEpiWarpsQ, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    BONES_CHECK(cudaFuncSetAttribute(gemm_mxfp8_pair_kernel<kEpiWarpsQ, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    BONES_CHECK(cudaFuncSetAttribute(gemm_mxfp8_pair_kernel<kEpiWarpsQ, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_set = true;
  }
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int pairs = sms / 2;
  const int base_tiles = batch * p.tiles_m * p.tiles_n;
  p.atomic = (atomic && f32out) ? 1 : 0;
  p.splits = splits;
  if (p.splits <= 0) {
    p.splits = 1;
    if (f32out && base_tiles < 4 * pairs && KB >= 16) {
      long long best = -1;
      for (int c = 1; c <= 32; ++c) {
        if (c > KB / 4) break;
        const long long waves = ((long long)base_tiles * c + pairs - 1) / pairs;
        const long long cost = waves * (((long long)KB + c - 1) / c + 8) + (c > 1 ? 2 * c : 0);
        if (best < 0 || cost < best) { best = cost; p.splits = c; }
      }
    }
  }
  if (p.splits > 1 && !f32out) p.splits = 1;
  if (p.splits > KB) p.splits = KB;
  const int total = base_tiles * p.splits;
  const int clusters = total < pairs ? total : pairs;
  const int variant = (Dq != nullptr ? 1 : 0) | (Dt != nullptr ? 2 : 0);
  const dim3 grid(2 * clusters), block(96 + 32 * kEpiWarpsQ);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (variant) {
    case 0: gemm_mxfp8_pair_kernel<kEpiWarpsQ, 0><<<grid, block, smem, st>>>(ta, tb, tsa, tsb, td, p); break;
    case 1: gemm_mxfp8_pair_kernel<kEpiWarpsQ, 1><<<grid, block, smem, st>>>(ta, tb, tsa, tsb, td, p); break;
    case 2: gemm_mxfp8_pair_kernel<kEpiWarpsQ, 2><<<grid, block, smem, st>>>(ta, tb, tsa, tsb, td, p); break;
    default: gemm_mxfp8_pair_kernel<kEpiWarpsQ, 3><<<grid, block, smem, st>>>(ta, tb, tsa, tsb, td, p); break;
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
