// bf16 GEMM on CTA pairs: `tcgen05.mma.cta_group::2` computes a 256 x 256 output tile on two SMs of one cluster.
//
//   D[b] = epilogue( alpha * A[b] * B[b]^T , R[b] )     same operand layouts and epilogues as gemm_bf16.cu
//
// Why pairs: with one CTA per 128 x 256 tile every SM pulls (128 + 256) x K operand bytes per tile out of L2 and the
// L2 -> SM path is what saturates first.  In a pair each CTA loads its own 128 rows of A and only *half* of the B tile
// (128 of the 256 rows); the pair's two tensor cores read both halves of B through the cluster's shared memory window,
// so each SM loads (128 + 128) x K bytes for the same 128 x 256 slice of output: one third less L2 traffic, no
// multicast copy involved.  Each CTA keeps its own 128 x 256 accumulator, double-buffered in its TMEM.
//
// Protocol (all waits bounded, see common.cuh):
//   producer thread (each CTA)  waits its own `empty[s]`, issues its TMA loads in the `.cta_group::2` form whose
//                               transaction bytes are credited to the *leader's* `full[s]`; the leader arrives with
//                               the expected byte count of both CTAs, the peer arrives remotely (mapa + mbarrier.arrive)
//   MMA thread (leader only)    waits `full[s]`, issues the pair MMAs, commits with `.multicast::cluster` so `empty[s]`
//                               (and at the end of a tile `tmem_full[a]`) fire in both CTAs
//   epilogue warps (each CTA)   wait their own `tmem_full[a]`, drain their 128 rows, arrive on the leader's
//                               `tmem_empty[a]` (16 warp arrivals per tile)
#include <cooperative_groups.h>

#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace bones {

enum Epi2 : int { E2_BF16 = 0, E2_BF16_RES = 1, E2_RELU2 = 2, E2_ACC_F32 = 3, E2_MUL_2SQRT = 4, E2_F32 = 5, E2_F32_RES = 6, E2_SOFTCAP = 7 };

struct Gemm2Params {
  int M, N, K, batch;
  int a_major, b_major;
  int epi;
  float alpha, beta;
  void* D;
  long long ldd, strideD;
  const void* R;
  long long ldr, strideR;
  int* err;
  int tiles_m, tiles_n;
  int splits;
  int atomic;          // E2_ACC_F32: always add with atomics (other GPUs add into the same buffer at the same time)
  int wide;            // rows are 32-byte aligned: use 256-bit global accesses in the epilogue
};

constexpr int PM = 256;      // pair tile M (128 per CTA)
constexpr int PN = 256;      // pair tile N (each CTA loads 128 rows of B)
constexpr int PK = 64;
constexpr int PSTAGES = 6;
constexpr uint32_t PA_BYTES = 128 * PK * 2;
constexpr uint32_t PB_BYTES = 128 * PK * 2;
constexpr uint32_t PSTAGE_BYTES = PA_BYTES + PB_BYTES;
constexpr int kGroupM2 = 8;

__device__ __forceinline__ void decode_tile2(int tile, int tiles_m, int tiles_n, int& b, int& mb, int& nb) {
  const int per_batch = tiles_m * tiles_n;
  b = tile / per_batch;
  const int rem = tile - b * per_batch;
  const int group_size = kGroupM2 * tiles_n;
  const int gid = rem / group_size;
  const int first_m = gid * kGroupM2;
  const int gsz = min(tiles_m - first_m, kGroupM2);
  const int in_group = rem - gid * group_size;
  mb = first_m + in_group % gsz;
  nb = in_group / gsz;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t local_bar, uint32_t cta) {
  asm volatile(
      "{\n"
      ".reg .b32 rem;\n"
      "mapa.shared::cluster.u32 rem, %0, %1;\n"
      "mbarrier.arrive.shared::cluster.b64 _, [rem];\n"
      "}\n" ::"r"(local_bar),
      "r"(cta)
      : "memory");
}
// Pair-mode TMA load: the destination is this CTA's shared memory, the transaction bytes go to the leader's barrier.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar & 0xFEFFFFFFu), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// commit that arrives on the barrier at the same shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
               : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(320, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t bars = base + PSTAGES * PSTAGE_BYTES;
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (PSTAGES + s); };
  auto tfull = [&](int a) { return bars + 8u * (2 * PSTAGES + a); };
  auto tempty = [&](int a) { return bars + 8u * (2 * PSTAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * PSTAGES + 4);
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + PSTAGES * PSTAGE_BYTES + 8 * (2 * PSTAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + PSTAGES * PSTAGE_BYTES + 8 * (2 * PSTAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(full(s), 2);        // leader: its own arrive.expect_tx + the peer's remote arrive
      mbar_init(empty(s), 1);       // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull(a), 1);       // one multicast commit
      mbar_init(tempty(a), 16);     // leader: 8 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  cluster_sync_all();               // barriers of both CTAs exist before anyone signals across the pair
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_g;

  // Work units are ordered K-split slowest: the pairs that run at one time work on the same K range of (nearly) all output
  // tiles, so every operand slice is fetched from DRAM once and shared through L2 by the tiles that need it.
  const int base_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int total = base_tiles * p.splits;
  const int KB = (p.K + PK - 1) / PK;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  // The producer and MMA roles run on all 32 lanes of their warp with warp-uniform state and issue from the elected lane
  // (see `elect_one` in common.cuh).  A lane whose bounded wait ran out turns `dead`: it walks the rest of the loops
  // without waiting or issuing, so the warp stays together for every `elect.sync` and reaches the tear-down as one.
  if (warp == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int tile = cluster_id; tile < total; tile += n_clusters) {
      int b, mb, nb;
      const int sp = p.splits == 1 ? 0 : tile / base_tiles;
      decode_tile2(tile - sp * base_tiles, p.tiles_m, p.tiles_n, b, mb, nb);
      const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
      const int m0 = mb * PM + (int)rank * 128, n0 = nb * PN + (int)rank * 128;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!dead) dead = !mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.err, ERR_WAIT_EMPTY);
        const uint32_t sa = base + stage * PSTAGE_BYTES, sb = sa + PA_BYTES;
        if (elect_one() && !dead) {
          if (leader) mbar_arrive_expect_tx(full(stage), 2 * PSTAGE_BYTES);
          if (p.a_major == 0) {
            tma_load_3d_pair(sa, &tma_a, full(stage), kb * PK, m0, b);
          } else {
            tma_load_3d_pair(sa, &tma_a, full(stage), m0, kb * PK, b);
            tma_load_3d_pair(sa + PK * 128, &tma_a, full(stage), m0 + 64, kb * PK, b);
          }
          if (p.b_major == 0) {
            tma_load_3d_pair(sb, &tma_b, full(stage), kb * PK, n0, b);
          } else {
            tma_load_3d_pair(sb, &tma_b, full(stage), n0, kb * PK, b);
            tma_load_3d_pair(sb + PK * 128, &tma_b, full(stage), n0 + 64, kb * PK, b);
          }
          if (!leader) mbar_arrive_cluster(full(stage), 0);
        }
        if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (leader) {
      const uint32_t idesc = umma_idesc_f16(PM, PN, 1, (uint32_t)p.a_major, (uint32_t)p.b_major);
      const uint32_t a_lbo = p.a_major ? PK * 128 : 0, b_lbo = p.b_major ? PK * 128 : 0;
      const uint32_t a_step = p.a_major ? (16 * 128) >> 4 : 32 >> 4;
      const uint32_t b_step = p.b_major ? (16 * 128) >> 4 : 32 >> 4;
      // descriptors of stage 0; a stage adds PSTAGE_BYTES >> 4 to the address field
      const uint64_t adesc0 = umma_smem_desc(base, a_lbo, 1024, kLayoutSw128);
      const uint64_t bdesc0 = umma_smem_desc(base + PA_BYTES, b_lbo, 1024, kLayoutSw128);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool dead = false;
      for (int tile = cluster_id; tile < total; tile += n_clusters) {
        if (!dead) dead = !mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * PN;
        const int sp = p.splits == 1 ? 0 : tile / base_tiles;
        const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!dead) dead = !mbar_wait(full(stage), phase, abort_flag, p.err, ERR_WAIT_FULL);
          tc_fence_after();
          const uint64_t soff = (uint64_t)(stage * (PSTAGE_BYTES >> 4));
          const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
          if (elect_one() && !dead) {
#pragma unroll
            for (int k = 0; k < PK / 16; ++k)
              umma_f16_pair(d_tmem, adesc + (uint64_t)(k * a_step), bdesc + (uint64_t)(k * b_step), idesc, ((kb - kb0) | k) ? 1u : 0u);
            tc_commit_pair(empty(stage));
            if (kb == kb1 - 1) tc_commit_pair(tfull(acc));
          }
          if (++stage == PSTAGES) { stage = 0; phase ^= 1u; }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // eight epilogue warps: two per 32-lane TMEM quadrant, each draining four of the tile's eight 32-column chunks
    const int q = warp & 3, half = (warp - 2) >> 2;
    const bool need_r = p.epi == E2_BF16_RES || p.epi == E2_MUL_2SQRT;
    const bool f32out = p.epi == E2_ACC_F32 || p.epi == E2_F32 || p.epi == E2_F32_RES;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cluster_id; tile < total; tile += n_clusters) {
      int b, mb, nb;
      decode_tile2(tile % base_tiles, p.tiles_m, p.tiles_n, b, mb, nb);
      const int row = mb * PM + (int)rank * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long drow = (long long)b * p.strideD + (long long)row * p.ldd;
      const long long rrow = (long long)b * p.strideR + (long long)row * p.ldr;
      // the residual / auxiliary operand of this thread's four chunks is fetched before the accumulator is awaited, so
      // its latency hides behind the tile's MMAs
      uint4 rpre[4][4];
      const bool pre = need_r && p.wide && row_ok;
      if (pre) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int col0 = nb * PN + (half * 4 + cc) * 32;
          if (col0 + 32 <= p.N) {
            const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.R) + rrow + col0;
            ld_global_v8(R, rpre[cc][0], rpre[cc][1]);
            ld_global_v8(R + 16, rpre[cc][2], rpre[cc][3]);
          }
        }
      }
      const bool got = mbar_wait(tfull(acc), acc_phase, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int c = half * 4 + cc;
        uint32_t r[32];
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * PN + c * 32);
        __syncwarp();
        BONES_TMEM_LD32(taddr, r);
        tmem_ld_wait();
        const int col0 = nb * PN + c * 32;
        if (row_ok && col0 < p.N) {
          const size_t esz = f32out ? 4 : 2;
          gemm_store_chunk(r, p.epi, p.alpha, p.beta, p.wide != 0, p.splits > 1 || p.atomic, reinterpret_cast<uint8_t*>(p.D) + (drow + col0) * esz,
                           reinterpret_cast<const uint8_t*>(p.R) + (rrow + col0) * esz, pre && col0 + 32 <= p.N, rpre[cc],
                           min(32, p.N - col0));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty(acc), 0);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // tear-down: both CTAs of the pair always arrive here (every wait above is bounded)
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

static int operand_tmap2(CUtensorMap* out, const void* ptr, int major, long long rows, long long K, long long ld, long long stride,
                         int batch) {
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  if (major == 0) {
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)rows;
    box[0] = PK; box[1] = 128;
  } else {
    dims[0] = (uint64_t)rows; dims[1] = (uint64_t)K;
    box[0] = 64; box[1] = PK;
  }
  dims[2] = (uint64_t)batch;
  box[2] = 1;
  strides[0] = (uint64_t)ld * 2;
  strides[1] = batch > 1 ? (uint64_t)stride * 2 : strides[0] * dims[1];
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace bones

extern "C" {

int bones_gemm_bf16_pair(const void* A, const void* B, void* D, const void* R, int M, int N, int K, int batch, long long lda,
                         long long ldb, long long ldd, long long ldr, long long strideA, long long strideB, long long strideD,
                         long long strideR, int a_major, int b_major, int epi, float alpha, float beta, int splits, int atomic, void* stream) {
  using namespace bones;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)D & 15)) return -2;
  const bool f32out = epi == E2_ACC_F32 || epi == E2_F32 || epi == E2_F32_RES;
  if (ldd % (f32out ? 4 : 8)) return -3;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_major = a_major; p.b_major = b_major; p.epi = epi;
  p.alpha = alpha; p.beta = beta;
  p.D = D; p.ldd = ldd; p.strideD = strideD;
  p.R = R ? R : D; p.ldr = R ? ldr : ldd; p.strideR = R ? strideR : strideD;
  p.err = error_word();
  const long long wal = f32out ? 8 : 16;     // elements per 32 bytes
  p.wide = ((ldd % wal == 0) && (strideD % wal == 0) && (!R || (ldr % wal == 0 && strideR % wal == 0)) && (((uintptr_t)D & 31) == 0) &&
            (!R || ((uintptr_t)R & 31) == 0)) ? 1 : 0;
  p.tiles_m = (M + PM - 1) / PM;
  p.tiles_n = (N + PN - 1) / PN;
  CUtensorMap ta, tb;
  int rc = operand_tmap2(&ta, A, a_major, M, K, lda, strideA, batch);
  if (rc) return rc;
  rc = operand_tmap2(&tb, B, b_major, N, K, ldb, strideB, batch);
  if (rc) return rc;
  constexpr size_t smem = (size_t)PSTAGES * PSTAGE_BYTES + 8 * (2 * PSTAGES + 4) + 16 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int pairs = sms / 2;
  const int base_tiles = batch * p.tiles_m * p.tiles_n;
  const int KB = (K + PK - 1) / PK;
  p.atomic = (atomic && epi == E2_ACC_F32) ? 1 : 0;
  p.splits = splits;
  if (p.splits <= 0) {
    p.splits = 1;
    if (epi == E2_ACC_F32 && base_tiles < 4 * pairs && KB >= 32) {
      long long best = -1;
      for (int c = 1; c <= 32; ++c) {
        if (c > KB / 8) break;
        const long long waves = ((long long)base_tiles * c + pairs - 1) / pairs;
        const long long cost = waves * (((long long)KB + c - 1) / c + 6) + (c > 1 ? 2 * c : 0);
        if (best < 0 || cost < best) { best = cost; p.splits = c; }
      }
    }
  }
  if (p.splits > 1 && epi != E2_ACC_F32) p.splits = 1;
  if (p.splits > KB) p.splits = KB;          // every split owns at least one K block (its last block signals the epilogue)
  const int total = base_tiles * p.splits;
  const int clusters = total < pairs ? total : pairs;
  gemm_bf16_pair_kernel<<<2 * clusters, 320, smem, reinterpret_cast<cudaStream_t>(stream)>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

}  // extern "C"
