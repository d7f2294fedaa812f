/* Allocation-free entry point of libbones_b200.so.
 *
 * This entry point has no counterpart in the reference project; it exists for callers of this library that are not
 * allowed to allocate device memory while they run: code executing inside a region where cudaMalloc is forbidden or
 * would deadlock (a real-time inference loop with a frozen memory plan, a plug-in hosted by a process that owns the
 * allocator, an allocator callback), and embedders that do not link PyTorch at all and therefore have no caching
 * allocator to borrow scratch from.
 *
 * bones_attn_bwd_noalloc computes exactly what bones_attn_delta + bones_attn_bwd compute (the attention backward
 * for head_dim 128: dq-hat accumulated into the first half of `dqk`, dk-hat written to its second half, dv written to
 * `dv`) but keeps its only scratch -- delta[b,h,t] = sum_d dO*O, B*H*T floats -- in a fixed 4 MiB __device__ array
 * inside the library instead of taking it from the caller.  It calls no cudaMalloc, cudaFree or allocating library
 * routine.  Every GPU that loads the library holds those 4 MiB until the process exits.
 *
 *   limit      B * H * T <= 1,048,576.  Larger problems are refused with -10 (see bones_attn_bwd_noalloc_strerror).
 *   first call the first call on each device resolves the scratch symbol's device address (cudaGetSymbolAddress) and
 *              raises the kernel's shared-memory limit; make that first call before any stream capture on the device.
 *              The set-up is guarded by a mutex, so two host threads may race to make it; only the set-up is guarded,
 *              the scratch itself is not (see "sharing").
 *   errors     every wait inside the kernel is bounded.  If one runs out (it should not: it would mean a lost TMA or MMA
 *              completion) the kernel stops early, leaves `dqk` / `dv` incomplete and records a code in an error word
 *              that belongs to this entry point alone; the call has returned 0 long before, because launches are
 *              asynchronous.  Read it with bones_attn_bwd_noalloc_error_read_clear(stream) after the calls whose
 *              results you are about to use: it waits for the stream, returns 0 or the first recorded code (1..7: which
 *              wait gave up) and clears the word.  It allocates nothing either.
 *   sharing    all calls on a device share the one scratch array, and it keeps the previous call's contents.  The
 *              range a call uses is fully rewritten before it is read, and the dq-hat half of `dqk` is zeroed by the
 *              call itself, so back-to-back calls on one stream are safe.  Two calls that can overlap on the GPU
 *              (different streams, no ordering between them) race on the scratch: serialise them.
 *   inputs     qk  [B*T, 2*H*128] bf16 (rotated, normalised q | k)      qkv [B*T, 3*H*128] bf16 (v read in place)
 *              dy, y [B*T, H*128] bf16      lse [B,H,T] f32      doc_start [B,T] int32 or NULL
 *   outputs    dqk [B*T, 2*H*128] f32       dv [B*T, H*128] bf16
 *   returns    0, a negative argument/set-up code, or a positive cudaError_t.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int bones_attn_bwd_noalloc(const void* qk, const void* qkv, const void* dy, const void* y, const float* lse, float* dqk,
                           void* dv, const int* doc_start, int B, int T, int H, float scale, int window_tiles,
                           void* stream);
int bones_attn_bwd_noalloc_error_read_clear(void* stream);
const char* bones_attn_bwd_noalloc_strerror(int code);
#ifdef __cplusplus
}
#endif
