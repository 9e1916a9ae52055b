// ErrorMonitor: a host thread that watches the device status blocks while kernels run.
//
// Kernels of this library never trap: a wait that runs out writes a record into a status block and the kernel
// returns.  Someone has to look at those blocks while the stream is still busy, and someone has to be able to raise
// the abort flag *past* a running kernel (a write queued on the kernel's own stream would wait behind it).  This
// thread does both on a stream of its own: every `interval_ms` it copies the registered blocks to pinned memory;
// the first non-zero code is kept as the report, the abort word of every registered block is raised so that all other
// bounded waits on this GPU give up at their next poll instead of after their full limit, and a flag that the host
// (and, through the stats block, other processes) can read is set.  It also raises the abort on request.
// Counterpart in the reference: the fault absorber and peer-termination watcher that halt a port instead of letting the
// process die (rdma/mesh-events.c:120-210), and the host's wait codes ETIMEDOUT / ECANCELED (rdma/mesh.h:15-17).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>
#include <cuda_runtime.h>
#include "../device/status.cuh"
#include "host_common.h"

namespace {

struct Monitor {
  int device = 0, interval_ms = 5;
  std::vector<mesh::Status*> blocks;
  std::thread th;
  std::atomic<bool> run{true};
  std::atomic<int> abort_request{0};
  std::atomic<int> seen_error{0};
  std::atomic<uint64_t> polls{0};
  std::mutex mu;
  mesh::Status first{};            // first failing record
  int first_block = -1;
  int cuda_error = 0;
};

void raise_abort_all(Monitor* m, cudaStream_t s, int* pinned_one) {
  *pinned_one = 1;
  for (mesh::Status* b : m->blocks)
    cudaMemcpyAsync(reinterpret_cast<char*>(b) + offsetof(mesh::Status, abort), pinned_one, sizeof(int), cudaMemcpyHostToDevice, s);
  cudaStreamSynchronize(s);
}

void loop(Monitor* m) {
  if (cudaSetDevice(m->device) != cudaSuccess) { m->cuda_error = 1; return; }
  cudaStream_t s;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { m->cuda_error = 2; return; }
  mesh::Status* pinned = nullptr;
  int* one = nullptr;
  const size_t n = m->blocks.size();
  if (cudaMallocHost(&pinned, sizeof(mesh::Status) * (n ? n : 1)) != cudaSuccess ||
      cudaMallocHost(&one, sizeof(int)) != cudaSuccess) { m->cuda_error = 3; cudaStreamDestroy(s); return; }
  bool raised = false;
  while (m->run.load()) {
    for (size_t i = 0; i < n; ++i)
      cudaMemcpyAsync(pinned + i, m->blocks[i], sizeof(mesh::Status), cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) { m->cuda_error = 4; break; }
    m->polls.fetch_add(1);
    bool failing = false;
    for (size_t i = 0; i < n; ++i) {
      if (pinned[i].code != 0) {
        failing = true;
        if (!m->seen_error.load()) {
          std::lock_guard<std::mutex> lk(m->mu);
          m->first = pinned[i];
          m->first_block = (int)i;
          m->seen_error.store(1);
        }
      }
    }
    if ((failing || m->abort_request.load()) && !raised) {
      raise_abort_all(m, s, one);
      raised = true;
    }
    if (!failing && !m->abort_request.load()) raised = false;       // cleared by the host: arm again
    std::this_thread::sleep_for(std::chrono::milliseconds(m->interval_ms));
  }
  cudaFreeHost(pinned);
  cudaFreeHost(one);
  cudaStreamDestroy(s);
}

}  // namespace

extern "C" {

typedef struct MeshMonitorReport {
  int seen_error, block_index, cuda_error, pad;
  unsigned long long polls;
  int code, site, block, thread;
  unsigned long long expected, seen, aux;
} MeshMonitorReport;

void* mesh_monitor_start(int device, void** status_blocks, int n, int interval_ms) {
  auto* m = new Monitor();
  m->device = device;
  m->interval_ms = interval_ms > 0 ? interval_ms : 5;
  for (int i = 0; i < n; ++i) m->blocks.push_back(reinterpret_cast<mesh::Status*>(status_blocks[i]));
  m->th = std::thread(loop, m);
  return m;
}

// Raise (1) or withdraw (0) the host's abort request; the monitor writes the blocks' abort words on its own stream.
void mesh_monitor_abort(void* h, int v) { reinterpret_cast<Monitor*>(h)->abort_request.store(v); }

// Forget the recorded failure (after the host has handled it and cleared the device blocks).
void mesh_monitor_clear(void* h) {
  auto* m = reinterpret_cast<Monitor*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  m->seen_error.store(0);
  m->first_block = -1;
  memset(&m->first, 0, sizeof(m->first));
}

void mesh_monitor_report(void* h, MeshMonitorReport* out) {
  auto* m = reinterpret_cast<Monitor*>(h);
  std::lock_guard<std::mutex> lk(m->mu);
  out->seen_error = m->seen_error.load();
  out->block_index = m->first_block;
  out->cuda_error = m->cuda_error;
  out->polls = m->polls.load();
  out->code = m->first.code; out->site = m->first.site; out->block = m->first.block; out->thread = m->first.thread;
  out->expected = m->first.expected; out->seen = m->first.seen; out->aux = m->first.aux;
}

void mesh_monitor_stop(void* h) {
  auto* m = reinterpret_cast<Monitor*>(h);
  m->run.store(false);
  if (m->th.joinable()) m->th.join();
  delete m;
}

}  // extern "C"
