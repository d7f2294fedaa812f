// Persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores.
//
//   D[b] = epilogue( alpha * A[b] * B[b]^T , R[b] )       A: logical [M, K]   B: logical [N, K]   D, R: [M, N] row-major
//
// Either operand may be stored K-major (K contiguous; `x @ W^T` with both row-major) or MN-major (the M / N index
// contiguous; lets `dX = dY @ W` and `dW = dY^T @ X` run with no transposed copy).  One CTA per SM walks output tiles of
// 128 x BN:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles (128-byte swizzle) into a ring of shared-memory stages
//   warp 1      allocates TMEM; lane 0 issues tcgen05.mma (kind::f16, fp32 accumulate) and commits to mbarriers
//   warps 2-5   epilogue: tcgen05.ld the accumulator (double-buffered in TMEM so the next tile's MMAs overlap), apply
//               the epilogue and store
// Epilogues cover every dense use in the model: plain / residual add (alpha*acc + beta*R), ReLU^2, fp32 accumulate into
// a gradient buffer (weight gradients land directly in the optimizer's reduce-scatter slab), and the ReLU^2 backward
// `acc * 2*sqrt(h)` fused into the dX GEMM.
//
// Replaces the reference's bf16 GEMM primitives (round1/source/train.py:926-1052) and fused ReLU^2 MLP GEMMs
// (round2/source/kernels/nki_mlp_fused.py) with one tcgen05 kernel.
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace bones {

enum Epi : int {
  EPI_BF16 = 0,        // D(bf16) = alpha*acc
  EPI_BF16_RES = 1,    // D(bf16) = alpha*acc + beta*R(bf16)
  EPI_RELU2 = 2,       // D(bf16) = relu(alpha*acc)^2
  EPI_ACC_F32 = 3,     // D(f32) += alpha*acc
  EPI_MUL_2SQRT = 4,   // D(bf16) = alpha*acc * 2*sqrt(R(bf16))
  EPI_F32 = 5,         // D(f32)  = alpha*acc
  EPI_F32_RES = 6,     // D(f32)  = alpha*acc + beta*R(f32)
  EPI_SOFTCAP = 7,     // D(bf16) = beta * tanh(alpha*acc)
};

struct GemmParams {
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
  int wide;            // rows are 32-byte aligned: use 256-bit global accesses in the epilogue
  int splits;          // split-K factor (> 1 only with EPI_ACC_F32: partial tiles are added with vector atomics)
  int atomic;          // EPI_ACC_F32: always add with atomics (other GPUs add into the same buffer at the same time)
};

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGroupM = 8;

__device__ __forceinline__ void decode_tile(int tile, int tiles_m, int tiles_n, int& b, int& mb, int& nb) {
  const int per_batch = tiles_m * tiles_n;
  b = tile / per_batch;
  int rem = tile - b * per_batch;
  const int group_size = kGroupM * tiles_n;
  const int gid = rem / group_size;
  const int first_m = gid * kGroupM;
  const int gsz = min(tiles_m - first_m, kGroupM);
  const int in_group = rem - gid * group_size;
  mb = first_m + in_group % gsz;
  nb = in_group / gsz;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;   // 256 or 512: power of two

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_g = reinterpret_cast<volatile uint32_t*>(gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + STAGES * STAGE_BYTES + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull(a), 1);
      mbar_init(tempty(a), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_g;

  // K-split slowest: CTAs running at one time share a K range, so operand slices are reused through L2
  const int base_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int total = base_tiles * p.splits;
  const int KB = (p.K + BK - 1) / BK;

  // The producer and MMA roles run on all 32 lanes of their warp with warp-uniform state and issue from the elected lane
  // (see `elect_one` in common.cuh).  A lane whose bounded wait ran out turns `dead`: it walks the rest of the loops
  // without waiting or issuing, so the warp stays together for every `elect.sync`.
  if (warp == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      int b, mb, nb;
      const int sp = p.splits == 1 ? 0 : tile / base_tiles;
      decode_tile(tile - sp * base_tiles, p.tiles_m, p.tiles_n, b, mb, nb);
      const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!dead) dead = !mbar_wait(empty(stage), phase ^ 1u, abort_flag, p.err, ERR_WAIT_EMPTY);
        const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
        if (elect_one() && !dead) {
          mbar_arrive_expect_tx(full(stage), STAGE_BYTES);
          if (p.a_major == 0) {
            tma_load_3d(sa, &tma_a, full(stage), kb * BK, mb * BM, b);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_3d(sa + i * (BK * 128), &tma_a, full(stage), mb * BM + i * 64, kb * BK, b);
          }
          if (p.b_major == 0) {
            tma_load_3d(sb, &tma_b, full(stage), kb * BK, nb * BN, b);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_3d(sb + i * (BK * 128), &tma_b, full(stage), nb * BN + i * 64, kb * BK, b);
          }
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    const uint32_t idesc = umma_idesc_f16(BM, BN, 1, (uint32_t)p.a_major, (uint32_t)p.b_major);
    const uint32_t a_lbo = p.a_major ? BK * 128 : 0, b_lbo = p.b_major ? BK * 128 : 0;
    const uint32_t a_step = p.a_major ? (16 * 128) >> 4 : 32 >> 4;   // descriptor address units of 16 bytes per UMMA_K
    const uint32_t b_step = p.b_major ? (16 * 128) >> 4 : 32 >> 4;
    // descriptors of stage 0; a stage adds STAGE_BYTES >> 4 to the address field
    const uint64_t adesc0 = umma_smem_desc(base, a_lbo, 1024, kLayoutSw128);
    const uint64_t bdesc0 = umma_smem_desc(base + A_BYTES, b_lbo, 1024, kLayoutSw128);
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      if (!dead) dead = !mbar_wait(tempty(acc), acc_phase ^ 1u, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
      tc_fence_after();
      const uint32_t d_tmem = tmem + acc * BN;
      const int sp = p.splits == 1 ? 0 : tile / base_tiles;
      const int kb0 = p.splits == 1 ? 0 : (int)((long long)KB * sp / p.splits), kb1 = p.splits == 1 ? KB : (int)((long long)KB * (sp + 1) / p.splits);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!dead) dead = !mbar_wait(full(stage), phase, abort_flag, p.err, ERR_WAIT_FULL);
        tc_fence_after();
        const uint64_t soff = (uint64_t)(stage * (STAGE_BYTES >> 4));
        const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
        if (elect_one() && !dead) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16(d_tmem, adesc + (uint64_t)(k * a_step), bdesc + (uint64_t)(k * b_step), idesc, ((kb - kb0) | k) ? 1u : 0u);
          tc_commit(empty(stage));
          if (kb == kb1 - 1) tc_commit(tfull(acc));
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    const int q = warp & 3;
    const bool f32out = p.epi == EPI_ACC_F32 || p.epi == EPI_F32 || p.epi == EPI_F32_RES;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
      int b, mb, nb;
      decode_tile(tile % base_tiles, p.tiles_m, p.tiles_n, b, mb, nb);
      const bool got = mbar_wait(tfull(acc), acc_phase, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) break;   // warp-uniform: the TMEM loads below need the whole warp
      tc_fence_after();
      const int row = mb * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long drow = (long long)b * p.strideD + (long long)row * p.ldd;
      const long long rrow = (long long)b * p.strideR + (long long)row * p.ldr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 32);
        __syncwarp();
        BONES_TMEM_LD32(taddr, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c * 32;
        if (row_ok && col0 < p.N) {
          const size_t esz = f32out ? 4 : 2;
          const uint4 none[4] = {};
          gemm_store_chunk(r, p.epi, p.alpha, p.beta, p.wide != 0, p.splits > 1 || p.atomic, reinterpret_cast<uint8_t*>(p.D) + (drow + col0) * esz,
                           reinterpret_cast<const uint8_t*>(p.R) + (rrow + col0) * esz, false, none, min(32, p.N - col0));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // tear-down: every role falls through to here, also after a bounded wait gave up
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the CTA's shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 8 * (2 * STAGES + 4) + 16 + 1024;
  static bool attr_done = false;
  if (!attr_done) {
    BONES_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  int dev = 0, sms = 0;
  BONES_CHECK(cudaGetDevice(&dev));
  BONES_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int base_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int KB = (p.K + BK - 1) / BK;
  if (p.splits <= 0) {
    // split-K only pays for fp32-accumulating outputs (weight gradients: few output tiles, very long K)
    p.splits = 1;
    if (p.epi == EPI_ACC_F32 && base_tiles < 4 * sms && KB >= 32) {
      long long best = -1;
      for (int c = 1; c <= 32; ++c) {
        if (c > KB / 8) break;
        const long long waves = ((long long)base_tiles * c + sms - 1) / sms;
        const long long cost = waves * (((long long)KB + c - 1) / c + 6) + (c > 1 ? 2 * c : 0);   // +6: tile prologue/epilogue, 2c: atomics
        if (best < 0 || cost < best) { best = cost; p.splits = c; }
      }
    }
  }
  if (p.splits > 1 && p.epi != EPI_ACC_F32) p.splits = 1;
  if (p.splits > KB) p.splits = KB;          // every split owns at least one K block (its last block signals the epilogue)
  const int total = base_tiles * p.splits;
  const int grid = total < sms ? total : sms;
  gemm_bf16_kernel<BN, STAGES><<<grid, 192, smem, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

static int operand_tmap(CUtensorMap* out, const void* ptr, int major, long long rows, long long K, long long ld, long long stride,
                        int batch, int box_rows) {
  // K-major: memory [rows][K], ld = elements between rows.   MN-major: memory [K][rows], ld = elements between k-rows.
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  if (major == 0) {
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)rows;
    box[0] = BK; box[1] = (uint32_t)box_rows;
  } else {
    dims[0] = (uint64_t)rows; dims[1] = (uint64_t)K;
    box[0] = 64; box[1] = BK;
  }
  dims[2] = (uint64_t)batch;
  box[2] = 1;
  strides[0] = (uint64_t)ld * 2;
  strides[1] = batch > 1 ? (uint64_t)stride * 2 : strides[0] * dims[1];
  return make_tmap(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace bones

extern "C" {

// Returns 0 on success, a CUDA error code (> 0) or a negative descriptor-encoding error.
int bones_gemm_bf16(const void* A, const void* B, void* D, const void* R, int M, int N, int K, int batch, long long lda,
                    long long ldb, long long ldd, long long ldr, long long strideA, long long strideB, long long strideD,
                    long long strideR, int a_major, int b_major, int epi, float alpha, float beta, int force_bn, int splits, int atomic, void* stream) {
  using namespace bones;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)D & 15)) return -2;
  const bool f32out = epi == EPI_ACC_F32 || epi == EPI_F32 || epi == EPI_F32_RES;
  if (ldd % (f32out ? 4 : 8)) return -3;
  int bn = force_bn ? force_bn : (N > 128 ? 256 : 128);
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_major = a_major; p.b_major = b_major; p.epi = epi;
  p.alpha = alpha; p.beta = beta;
  p.D = D; p.ldd = ldd; p.strideD = strideD;
  p.R = R ? R : D; p.ldr = R ? ldr : ldd; p.strideR = R ? strideR : strideD;
  p.err = error_word();
  const long long wal = f32out ? 8 : 16;     // elements per 32 bytes
  p.wide = ((ldd % wal == 0) && (strideD % wal == 0) && (!R || (ldr % wal == 0 && strideR % wal == 0)) && (((uintptr_t)D & 31) == 0) &&
            (!R || ((uintptr_t)R & 31) == 0)) ? 1 : 0;
  p.splits = splits;
  p.atomic = (atomic && epi == EPI_ACC_F32) ? 1 : 0;
  CUtensorMap ta, tb;
  int rc = operand_tmap(&ta, A, a_major, M, K, lda, strideA, batch, BM);
  if (rc) return rc;
  rc = operand_tmap(&tb, B, b_major, N, K, ldb, strideB, batch, bn);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 256) return launch_gemm<256, 4>(ta, tb, p, s);
  return launch_gemm<128, 6>(ta, tb, p, s);
}

}  // extern "C"
