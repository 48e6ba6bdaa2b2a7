// CUDA-graph capture / replay of one training step, plus small runtime queries.
// The executor captures its launch sequence once per feed shape (all buffers come
// from a static plan, so every kernel argument is stable) and replays it, which
// removes the per-node host work from the steady state.
#include <cuda_runtime.h>
#include <stdint.h>

#define TSB_OK 0
#define TSB_ERR_ARG 1
#define TSB_ERR_LAUNCH 3

namespace {
int rc(cudaError_t e) { return e == cudaSuccess ? TSB_OK : (TSB_ERR_LAUNCH | ((int)e << 8)); }
}

extern "C" {

int tsb_graph_begin(void* stream) {
  return rc(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeRelaxed));
}

// Ends the capture and instantiates; *exec_out receives an opaque handle.
int tsb_graph_end(void* stream, void** exec_out) {
  if (!exec_out) return TSB_ERR_ARG;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph);
  if (e != cudaSuccess) {
    cudaGetLastError();   // an invalidated capture is over now; the next launch's error check must not see it
    return rc(e);
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return rc(e);
  *exec_out = exec;
  return TSB_OK;
}

int tsb_graph_launch(void* exec, void* stream) {
  return rc(cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec), static_cast<cudaStream_t>(stream)));
}

int tsb_graph_destroy(void* exec) { return rc(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec))); }

// Stream-ordering and copy actions as entries of their own, so that a recorded step (csrc/runtime/step_tape.cc)
// replays them like any kernel entry.  `event` is a cudaEvent_t the caller owns.
int tsb_event_record(void* event, void* stream) {
  if (!event) return TSB_ERR_ARG;
  return rc(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
}

int tsb_stream_wait_event(void* stream, void* event) {
  if (!event) return TSB_ERR_ARG;
  return rc(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
}

// Byte copy between device memory and page-locked host memory (either direction) on `stream`.
int tsb_memcpy_async(void* dst, const void* src, long long bytes, void* stream) {
  if (!dst || !src || bytes < 0) return TSB_ERR_ARG;
  if (bytes == 0) return TSB_OK;
  return rc(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
}

// free / total device memory in bytes
int tsb_mem_info(long long* free_b, long long* total_b) {
  size_t f = 0, t = 0;
  cudaError_t e = cudaMemGetInfo(&f, &t);
  if (free_b) *free_b = (long long)f;
  if (total_b) *total_b = (long long)t;
  return rc(e);
}

}  // extern "C"
