// Norm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project (which always works through torch's allocator);
// it exists for users of this library who call it from places where allocating is not an option:
//
//   * C or C++ programs that link libhg_sm100.so directly and have no tensor allocator at hand;
//   * jobs whose device memory is planned to the last byte before training starts (a 180 GB part filled by a
//     memory-aware parallelism plan), where a transient buffer taken in the middle of a backward pass could be the
//     allocation that fails;
//   * code running while the process's allocator is locked or must stay untouched -- inside an allocator callback,
//     an out-of-memory handler, or a section whose memory pool is frozen.
//
// hg_norm_bwd needs a scratch buffer (per-CTA partial sums of the weight and bias gradients) that its caller
// allocates.  hg_norm_bwd_noalloc computes the same thing but keeps that scratch in a fixed array inside the
// library's device image, so the call itself performs no cudaMalloc / cudaFree and calls nothing that allocates.
//
// Limits and rules:
//   * H (the normalised width) must be a multiple of 8 and at most HG_NORM_NOALLOC_MAX_H; larger widths are
//     rejected with HG_NORM_NOALLOC_TOO_WIDE and nothing is launched.  The array holds
//     2 * HG_NORM_NOALLOC_PARTS * HG_NORM_NOALLOC_MAX_H floats (9.25 MiB per device).
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current) and remembers it.  Make that first call during start-up, outside any stream capture.
//   * All calls on a device share the one array.  Two calls whose kernels can overlap (different streams without an
//     ordering between them, or different host threads) race on it and give wrong gradients: order them.
//   * The array keeps whatever the last call left in it.  Nothing has to be cleared between calls: each call
//     overwrites every scratch row that it later reads.
//   * Arguments other than the scratch are those of hg_norm_bwd: bf16 dy / h / w / dres / dx, fp32 rstd / mean /
//     dw / db; `mean` and `db` are null for RMSNorm; `dres` may be null; `accumulate` != 0 adds into dw / db.
//
//   * dy, h, w, rstd, dx and dw must not be null, nor `mean` for LayerNorm (rms == 0): a null one is rejected with
//     HG_NORM_NOALLOC_NULL_ARG before anything is launched (the kernel would read or write through it).
//   * The per-device address cache has HG_NORM_NOALLOC_MAX_DEVICES entries: a call made with a current device
//     index at or beyond that is rejected with HG_NORM_NOALLOC_BAD_DEVICE.
//
// Returns 0 on success, -1 for a bad shape (H not a positive multiple of 8), HG_NORM_NOALLOC_TOO_WIDE for H beyond
// the maximum, HG_NORM_NOALLOC_NULL_ARG, HG_NORM_NOALLOC_BAD_DEVICE, -(1000 + cudaError) when the address lookup
// fails, else the cudaError of the launches.
#pragma once

#define HG_NORM_NOALLOC_MAX_H 8192
#define HG_NORM_NOALLOC_PARTS 148
#define HG_NORM_NOALLOC_TOO_WIDE (-2)
#define HG_NORM_NOALLOC_NULL_ARG (-3)
#define HG_NORM_NOALLOC_BAD_DEVICE (-4)
#define HG_NORM_NOALLOC_MAX_DEVICES 64

#ifdef __cplusplus
extern "C" {
#endif

int hg_norm_bwd_noalloc(const void* dy, const void* h, const void* w, const void* rstd, const void* mean,
                        const void* dres, void* dx, void* dw, void* db, int rows, int H, int rms, int accumulate,
                        void* stream);

#ifdef __cplusplus
}
#endif
