/* One C entry point of the memarch B200 kernels that never allocates device memory.
 *
 * This function has no counterpart in the reference implementation.  It exists for callers that are not allowed to
 * call cudaMalloc (or anything that allocates behind their back, the PyTorch caching allocator included): code that
 * runs inside someone else's memory budget - a host application that hands this library a fixed arena, a process
 * whose device memory is fully reserved up front by another runtime, or a step replayed in an environment where an
 * allocation would fail or stall.  Such a caller owns every input and output buffer; the only extra memory the
 * optimizer step needs (row / column statistics of the homeostasis normalisation) lives in a fixed array inside the
 * library image.
 *
 *   memarch_instinct_hs_step_noalloc  -  one Instinct optimizer step with homeostasis ("hs") normalisation of a
 *   2-D weight (rows x cols, cols contiguous): momentum update, row -> column -> row normalisation of the update,
 *   weight decay, weight step.  Same maths and same kernels as the allocating path (`instinct_step` of the Python
 *   extension, kind "hs").
 *
 * Limits and rules
 *   - Scratch: a file-scope __device__ array of MEMARCH_NOALLOC_SCRATCH_FLOATS floats (4 MiB), present once on every
 *     GPU that loads the library until the process exits.  A call needs 3*pad4(rows) + 2*pad4(cols) + 4 floats of it
 *     (pad4 = rounded up to a multiple of 4; at most 3*rows + 2*cols + 19); larger problems are refused with
 *     MEMARCH_NOALLOC_TOO_LARGE and a message on stderr - nothing is launched.
 *   - Rows of more than 51 200 columns are refused the same way: the kernels stage one row of column scales
 *     (4 bytes per column) in shared memory and ask for at most 200 KB of it.
 *   - The first call on a device looks up the device address of that array (cudaGetSymbolAddress, with that device
 *     current) and keeps it.  Make this first call outside of any CUDA stream capture.
 *   - Every call uses the same array and the array keeps what the previous call left; the function clears the
 *     parts that must start at zero itself (cudaMemsetAsync on `stream`).  Two calls whose kernels can overlap on the
 *     GPU (different streams without ordering, or different host threads) race on the array: order them.
 *   - No cudaMalloc, cudaFree or allocating library routine is called; work is enqueued on `stream` and the function
 *     returns without synchronising.
 *   - cols must be a multiple of 4 and all pointers 16-byte aligned.
 */
#ifndef MEMARCH_NOALLOC_H_
#define MEMARCH_NOALLOC_H_

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MEMARCH_NOALLOC_SCRATCH_FLOATS (1 << 20)

#define MEMARCH_NOALLOC_OK 0
#define MEMARCH_NOALLOC_TOO_LARGE 1
#define MEMARCH_NOALLOC_BAD_ARG 2
#define MEMARCH_NOALLOC_CUDA_ERROR 3

/* weight / grad / momentum: device pointers, bf16 when the matching *_bf16 flag is non-zero, else fp32.
 * master: device pointer to the exact fp32 copy of a bf16 weight, or NULL (then the weight itself is stepped).
 * gain, stake, lr_scaled: the optimizer's per-step scalars (host values); step = lr_scaled * (1 + (gain-1)*stake).
 * weight_decay: already divided by the optimizer's `scale` (0 disables it).
 * Returns MEMARCH_NOALLOC_OK or one of the codes above. */
int memarch_instinct_hs_step_noalloc(void* weight, const void* grad, void* momentum, float* master, int weight_bf16,
                                     int grad_bf16, int momentum_bf16, long long rows, long long cols, float gain,
                                     float stake, float lr_scaled, float beta, float weight_decay, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
