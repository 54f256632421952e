// Non-blocking host view of the device status word: a 4-byte snapshot copy per poll plus an event that says when the
// copy has landed.  This is how an expired device-side wait reaches the caller without any synchronisation.
#include <mutex>

#include "../../include/coda_b200.h"
#include "gemm_host.cuh"

using namespace cb;

namespace {
constexpr int kMaxDevices = 64;

struct Snapshot {
  int* host = nullptr;  // pinned
  cudaEvent_t landed = nullptr;
  bool pending = false;
};

Snapshot g_snapshots[kMaxDevices];
std::mutex g_snapshot_mutex;
}  // namespace

extern "C" int coda_b200_status_poll(int* dev_status, void* stream_ptr) {
  if (dev_status == nullptr) return fail(kBadArgument, "device status word is required");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess) {
    (void)cudaGetLastError();  // e.g. the legacy stream while another stream captures: nothing may be enqueued now
    return kOk;
  }
  if (capture != cudaStreamCaptureStatusNone) return kOk;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return fail(kCudaError, "status poll: no current device");

  std::lock_guard<std::mutex> lock(g_snapshot_mutex);
  Snapshot& snap = g_snapshots[device];
  if (snap.host == nullptr) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&snap.host), sizeof(int), cudaHostAllocDefault) != cudaSuccess ||
        cudaEventCreateWithFlags(&snap.landed, cudaEventDisableTiming) != cudaSuccess) {
      snap.host = nullptr;
      return fail(kCudaError, std::string("status poll: ") + cudaGetErrorString(cudaGetLastError()));
    }
    *snap.host = 0;
  }
  if (snap.pending) {
    const cudaError_t q = cudaEventQuery(snap.landed);
    if (q == cudaErrorNotReady) return kOk;  // the copy is still behind queued work: look again at the next call
    if (q != cudaSuccess) return fail(kCudaError, std::string("status poll: ") + cudaGetErrorString(q));
    snap.pending = false;
    const int code = *snap.host;
    if (code != 0) {
      *snap.host = 0;
      if (cudaMemsetAsync(dev_status, 0, sizeof(int), stream) != cudaSuccess)
        return fail(kCudaError, std::string("status poll: ") + cudaGetErrorString(cudaGetLastError()));
      return code;
    }
  }
  if (cudaMemcpyAsync(snap.host, dev_status, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaEventRecord(snap.landed, stream) != cudaSuccess)
    return fail(kCudaError, std::string("status poll: ") + cudaGetErrorString(cudaGetLastError()));
  snap.pending = true;
  return kOk;
}
