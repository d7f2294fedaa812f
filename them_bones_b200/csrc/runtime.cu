// Host runtime shared by every kernel file: driver entry point for TMA descriptors, per-device error word, library
// version.  Exported C symbols are prefixed `bones_`.
#include <mutex>

#include "common.cuh"

namespace bones {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static int* g_err_words[64] = {nullptr};
static std::mutex g_err_mu;

int* error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_err_mu);
  if (!g_err_words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 64 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64 * sizeof(int));
    g_err_words[dev] = p;
  }
  return g_err_words[dev];
}

int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return -1;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

}  // namespace bones

extern "C" {

// Reads and clears the error word of the current device.  0 = no kernel gave up on a wait.
int bones_error_read_clear() {
  int* p = bones::error_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

int bones_version() { return 1; }

}  // extern "C"
