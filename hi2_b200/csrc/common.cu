// Error text of the calling thread and the ABI version.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace hi2 {
namespace {
thread_local char g_error[512] = "";
std::atomic<long long> g_launches{0};
}

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {
struct InFlight {
  cudaGraphExec_t exec;
  cudaEvent_t done;
};
std::mutex g_graph_mutex;
std::vector<InFlight> g_in_flight;
std::atomic<long long> g_graphs{0};

// Destroy the graphs whose completion event has passed (called outside any capture).
void retire_finished_graphs() {
  std::lock_guard<std::mutex> lock(g_graph_mutex);
  size_t keep = 0;
  for (size_t i = 0; i < g_in_flight.size(); ++i) {
    if (cudaEventQuery(g_in_flight[i].done) == cudaSuccess) {
      cudaGraphExecDestroy(g_in_flight[i].exec);
      cudaEventDestroy(g_in_flight[i].done);
    } else {
      g_in_flight[keep++] = g_in_flight[i];
    }
  }
  g_in_flight.resize(keep);
  (void)cudaGetLastError();  // cudaErrorNotReady of a pending event is not an error of the caller
}
}  // namespace

ChainGraph::ChainGraph(cudaStream_t stream) : stream_(stream) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return;  // the caller captures already: launch into the caller's graph
  }
  retire_finished_graphs();
  // thread-local mode: other threads of the process (a collective library's watchdog, another
  // device's driver thread) may go on calling the runtime while this thread captures
  capturing_ = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
  if (!capturing_) (void)cudaGetLastError();
}

ChainGraph::~ChainGraph() {
  if (capturing_) {  // finish() was not reached: drop what was captured
    cudaGraph_t g = nullptr;
    cudaStreamEndCapture(stream_, &g);
    if (g) cudaGraphDestroy(g);
    (void)cudaGetLastError();
  }
}

int ChainGraph::finish(int rc, const char* what) {
  if (!capturing_) return rc;
  capturing_ = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(stream_, &graph);
  if (e != cudaSuccess || graph == nullptr) {
    (void)cudaGetLastError();
    if (rc != HI2_OK) return rc;
    set_error("%s: stream capture failed: %s", what, cudaGetErrorString(e));
    return HI2_ERR_LAUNCH;
  }
  if (rc != HI2_OK) {
    cudaGraphDestroy(graph);
    return rc;
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    set_error("%s: graph instantiation failed: %s", what, cudaGetErrorString(e));
    return HI2_ERR_LAUNCH;
  }
  e = cudaGraphLaunch(exec, stream_);
  cudaEvent_t done = nullptr;
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&done, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventRecord(done, stream_);
  if (e != cudaSuccess) {
    set_error("%s: graph launch failed: %s", what, cudaGetErrorString(e));
    if (done) cudaEventDestroy(done);
    cudaStreamSynchronize(stream_);
    cudaGraphExecDestroy(exec);
    return HI2_ERR_LAUNCH;
  }
  g_graphs.fetch_add(1, std::memory_order_relaxed);
  std::lock_guard<std::mutex> lock(g_graph_mutex);
  g_in_flight.push_back({exec, done});
  return HI2_OK;
}
}  // namespace hi2

extern "C" int hi2_abi_version(void) { return 1; }
extern "C" const char* hi2_last_error(void) { return hi2::g_error; }
extern "C" long long hi2_launch_count(void) { return hi2::g_launches.load(std::memory_order_relaxed); }
extern "C" long long hi2_graph_launch_count(void) { return hi2::g_graphs.load(std::memory_order_relaxed); }
