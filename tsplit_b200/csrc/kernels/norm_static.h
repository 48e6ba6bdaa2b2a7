// tsb_bn_forward_static — batch-norm forward for callers that cannot allocate.
//
// This entry point has no counterpart in the reference; it exists for users of
// this library whose process must not (or cannot) obtain device memory while a
// step runs:
//   * a trainer that has handed the whole HBM budget to the capped activation
//     pool, so a lazy cudaMalloc inside the library would fail or push the
//     process over its budget;
//   * a latency-bound loop (serving, a real-time controller) where the implicit
//     device-wide synchronisation of cudaMalloc / cudaFree is not acceptable;
//   * a host that embeds the kernels under its own allocator and forbids the
//     library from touching the CUDA allocator at all.
// The regular entry point (tsb_bn_forward) keeps its column-statistics partial
// sums in a buffer it cudaMalloc's on first use.  This variant keeps them in a
// file-scope `static __device__` array inside the library image instead:
//   * size: 2 planes x 128 chunks x TSB_BN_STATIC_MAX_CHANNELS floats = 8 MiB,
//     held by every GPU that loads the library, until the process exits;
//   * limit: C <= TSB_BN_STATIC_MAX_CHANNELS, otherwise the call returns
//     error 7 ("size beyond the static scratch limit") and launches nothing;
//   * it calls no cudaMalloc, cudaFree or any allocating library routine; the
//     caller passes every input and output buffer.
// Set-up: the FIRST call on each device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it; make that
// first call before starting any stream capture.
// Sharing: all calls on a device use the same array.  Calls are safe back to
// back on one stream (each call rewrites every word it later reads, so stale
// contents from the previous call are never consumed and nothing needs
// clearing), but two calls that overlap on the GPU — different streams, or
// different host threads — race on it and must be serialised by the caller.
// Arguments and results are exactly those of tsb_bn_forward: x, y are
// [rows, C] views with row strides ldx / ldy (channels-last activations),
// save_mean / save_invstd / run_mean / run_var are [C], relu != 0 fuses a ReLU.
#pragma once

#define TSB_BN_STATIC_MAX_CHANNELS 8192

#ifdef __cplusplus
extern "C" {
#endif

int tsb_bn_forward_static(const float* x, const float* scale, const float* bias, float* y, float* save_mean,
                          float* save_invstd, float* run_mean, float* run_var, long long rows, long long C,
                          long long ldx, long long ldy, float momentum, float eps, int relu, void* stream);

#ifdef __cplusplus
}
#endif
