// Peer channels: one object per peer GPU with a state machine, a queue of transfers that are not issued from kernels,
// and one proxy thread per process that serves the queues.
//
// In the reference every port of the fabric is a child process with a command loop, spawned, driven through
// OPEN / MAKE / CONNECT / HALT / END and reaped by the bridge (rdma/mesh-children.c:73-242, rdma/mesh-child.c:44-191);
// a port that has outstanding work is flushed with a bounded wait before it leaves.  On NVLink the kernels move the
// data themselves, so what remains for a host-side channel is small: it knows whether the peer's memory is mapped
// (OPEN -> MAPPED -> CONNECTED -> HALTED -> CLOSED), it carries the few transfers that are better left to the copy
// engines (bulk copies of hundreds of megabytes that should not occupy SMs: checkpoint shards, re-sharding, weight
// broadcasts at start-up), cut into pieces so that progress can be observed, and it can be flushed with a time limit:
// only channels with outstanding work are waited for, and a channel whose work does not finish in time is HALTED,
// never waited for without bound.  With device == -1 the channel moves host memory with memcpy (no CUDA call at
// all), which is how the state machine, the queue and the flush are tested on machines without a GPU.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../runtime/host_common.h"

extern "C" void mesh_runtime_channel(int peer, int state);
extern "C" void mesh_runtime_count(int what, uint64_t n, int peer);

namespace mesh {
namespace {

enum ChannelState : int { CH_CLOSED = 0, CH_OPEN = 1, CH_MAPPED = 2, CH_CONNECTED = 3, CH_HALTED = 4 };
constexpr uint64_t PIECE = 64ull << 20;

struct Job {
  uint64_t ticket;
  void* dst;
  const void* src;
  uint64_t bytes;
  cudaEvent_t after;        // the channel stream waits for this event before the copy (nullptr: none)
};

struct Channel {
  int peer = -1;
  std::atomic<int> state{CH_OPEN};
  std::deque<Job> queue;                 // guarded by ChannelSet::mu
  cudaStream_t stream = nullptr;
  std::atomic<uint64_t> issued{0};       // highest ticket whose copies have been handed to the stream
  std::atomic<uint64_t> completed{0};    // highest ticket known complete
  std::vector<std::pair<uint64_t, cudaEvent_t>> events;   // (ticket, completion event), guarded by mu
  std::atomic<uint64_t> bytes{0};
};

struct ChannelSet {
  int rank, world, device;
  std::vector<Channel> ch;
  std::mutex mu;
  std::condition_variable cv;
  std::thread proxy;
  std::atomic<bool> run{true};
  std::atomic<uint64_t> next_ticket{1};

  void set_state(Channel& c, int s) {
    c.state.store(s);
    mesh_runtime_channel(c.peer, s);
  }

  // the proxy loop: take the oldest job of every connected channel in turn, issue it piece by piece
  void service() {
    if (device >= 0) cudaSetDevice(device);
    while (run.load()) {
      Job job{};
      Channel* owner = nullptr;
      {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait_for(lk, std::chrono::milliseconds(20), [&] {
          if (!run.load()) return true;
          for (auto& c : ch)
            if (!c.queue.empty() && c.state.load() == CH_CONNECTED) return true;
          return false;
        });
        if (!run.load()) break;
        for (auto& c : ch)
          if (!c.queue.empty() && c.state.load() == CH_CONNECTED) {
            job = c.queue.front();
            c.queue.pop_front();
            owner = &c;
            break;
          }
      }
      if (owner == nullptr) { poll(); continue; }
      bool ok = true;
      if (device < 0) {
        memcpy(job.dst, job.src, job.bytes);
        owner->completed.store(job.ticket);
      } else {
        if (job.after != nullptr) ok = cudaStreamWaitEvent(owner->stream, job.after, 0) == cudaSuccess;
        for (uint64_t off = 0; ok && off < job.bytes; off += PIECE) {
          const uint64_t n = job.bytes - off < PIECE ? job.bytes - off : PIECE;
          ok = cudaMemcpyAsync((char*)job.dst + off, (const char*)job.src + off, n, cudaMemcpyDefault, owner->stream) == cudaSuccess;
        }
        cudaEvent_t done = nullptr;
        if (ok) ok = cudaEventCreateWithFlags(&done, cudaEventDisableTiming) == cudaSuccess;
        if (ok) ok = cudaEventRecord(done, owner->stream) == cudaSuccess;
        if (ok) {
          std::lock_guard<std::mutex> lk(mu);
          owner->events.emplace_back(job.ticket, done);
        } else {
          (void)cudaGetLastError();
          set_state(*owner, CH_HALTED);
        }
      }
      owner->issued.store(job.ticket);
      owner->bytes.fetch_add(job.bytes);
      mesh_runtime_count(3, job.bytes, owner->peer);
      cv.notify_all();
      poll();
    }
  }

  // retire completion events that have fired
  void poll() {
    if (device < 0) return;
    std::lock_guard<std::mutex> lk(mu);
    for (auto& c : ch) {
      while (!c.events.empty()) {
        cudaError_t e = cudaEventQuery(c.events.front().second);
        if (e == cudaErrorNotReady) break;
        if (e == cudaSuccess) c.completed.store(c.events.front().first);
        else { (void)cudaGetLastError(); set_state(c, CH_HALTED); }
        cudaEventDestroy(c.events.front().second);
        c.events.erase(c.events.begin());
      }
    }
  }
};

}  // namespace
}  // namespace mesh

using namespace mesh;

extern "C" void* mesh_channels_create(int rank, int world, int device) {
  if (world < 1 || world > 64) { set_error(-2, "channels: world %d out of range", world); return nullptr; }
  auto* s = new ChannelSet();
  s->rank = rank; s->world = world; s->device = device;
  s->ch = std::vector<Channel>(world);
  for (int p = 0; p < world; ++p) {
    s->ch[p].peer = p;
    if (device >= 0) {
      cudaSetDevice(device);
      if (cudaStreamCreateWithFlags(&s->ch[p].stream, cudaStreamNonBlocking) != cudaSuccess) {
        set_error(-3, "channels: cannot create a stream for peer %d", p);
        delete s;
        return nullptr;
      }
    }
    mesh_runtime_channel(p, CH_OPEN);
  }
  s->proxy = std::thread([s] { s->service(); });
  return s;
}

// OPEN -> MAPPED -> CONNECTED, any -> HALTED, HALTED/any -> CLOSED.  Returns 0, or -1 for a transition out of order.
extern "C" int mesh_channel_advance(void* h, int peer, int to) {
  auto* s = (ChannelSet*)h;
  if (!s || peer < 0 || peer >= s->world) return set_error(-2, "channel: bad peer %d", peer);
  Channel& c = s->ch[peer];
  const int from = c.state.load();
  const bool ok = (to == CH_MAPPED && from == CH_OPEN) || (to == CH_CONNECTED && from == CH_MAPPED) ||
                  (to == CH_HALTED && from != CH_CLOSED) || (to == CH_CLOSED) || (to == CH_OPEN && from == CH_CLOSED);
  if (!ok) return set_error(-1, "channel %d: no transition from state %d to %d", peer, from, to);
  s->set_state(c, to);
  s->cv.notify_all();
  return 0;
}

extern "C" int mesh_channel_state(void* h, int peer) {
  auto* s = (ChannelSet*)h;
  return (!s || peer < 0 || peer >= s->world) ? -1 : s->ch[peer].state.load();
}

// Queue a copy on the channel to `peer`.  `after_stream` (device channels, may be NULL): the copy starts after the
// work that is on that stream now.  Returns the job's ticket (> 0), or 0 with an error text.
extern "C" uint64_t mesh_channel_copy(void* h, int peer, void* dst, const void* src, uint64_t bytes, void* after_stream) {
  auto* s = (ChannelSet*)h;
  if (!s || peer < 0 || peer >= s->world) { set_error(-2, "channel: bad peer %d", peer); return 0; }
  Channel& c = s->ch[peer];
  if (c.state.load() != CH_CONNECTED) { set_error(-5, "channel %d is not connected (state %d)", peer, c.state.load()); return 0; }
  Job j{};
  j.dst = dst; j.src = src; j.bytes = bytes;
  if (s->device >= 0 && after_stream != nullptr) {
    if (cudaEventCreateWithFlags(&j.after, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(j.after, (cudaStream_t)after_stream) != cudaSuccess) {
      set_error(-6, "channel %d: cannot record the ordering event", peer);
      return 0;
    }
  }
  {
    std::lock_guard<std::mutex> lk(s->mu);
    j.ticket = s->next_ticket.fetch_add(1);
    c.queue.push_back(j);
  }
  s->cv.notify_all();
  return j.ticket;
}

// 1 when the job has completed, 0 when not yet, -1 when the channel was halted before it could.
extern "C" int mesh_channel_done(void* h, int peer, uint64_t ticket) {
  auto* s = (ChannelSet*)h;
  if (!s || peer < 0 || peer >= s->world) return -1;
  s->poll();
  Channel& c = s->ch[peer];
  if (c.completed.load() >= ticket) return 1;
  return c.state.load() == CH_HALTED ? -1 : 0;
}

// Make `stream` wait (on the device) for the job; waits on the host, with a limit, until the proxy has issued it.
extern "C" int mesh_channel_wait_on_stream(void* h, int peer, uint64_t ticket, void* stream, int timeout_ms) {
  auto* s = (ChannelSet*)h;
  if (!s || peer < 0 || peer >= s->world) return set_error(-2, "channel: bad peer %d", peer);
  Channel& c = s->ch[peer];
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  {
    std::unique_lock<std::mutex> lk(s->mu);
    while (c.issued.load() < ticket) {
      if (c.state.load() == CH_HALTED) return set_error(-7, "channel %d halted", peer);
      if (s->cv.wait_until(lk, deadline) == std::cv_status::timeout && c.issued.load() < ticket)
        return set_error(110, "channel %d: job %llu was not issued within %d ms", peer, (unsigned long long)ticket, timeout_ms);
    }
  }
  if (s->device < 0) return 0;
  // everything issued so far on the channel stream precedes this marker
  cudaEvent_t e;
  MESH_CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  MESH_CUDA_OK(cudaEventRecord(e, c.stream));
  MESH_CUDA_OK(cudaStreamWaitEvent((cudaStream_t)stream, e, 0));
  MESH_CUDA_OK(cudaEventDestroy(e));
  return 0;
}

// Wait, with a limit, for the channels that have outstanding work (and only for those).  A channel that does not
// finish in time is HALTED.  Returns the number of channels halted by this call.
extern "C" int mesh_channels_flush(void* h, int timeout_ms) {
  auto* s = (ChannelSet*)h;
  if (!s) return 0;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int halted = 0;
  for (auto& c : s->ch) {
    while (true) {
      uint64_t last = 0;
      bool pending;
      {
        std::lock_guard<std::mutex> lk(s->mu);
        pending = !c.queue.empty();
        last = c.issued.load();
      }
      s->poll();
      if (!pending && c.completed.load() >= last) break;
      if (c.state.load() != CH_CONNECTED) break;                 // nothing will move on a channel that is not up
      if (std::chrono::steady_clock::now() > deadline) {
        s->set_state(c, CH_HALTED);
        ++halted;
        break;
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
  }
  return halted;
}

extern "C" uint64_t mesh_channel_bytes(void* h, int peer) {
  auto* s = (ChannelSet*)h;
  return (!s || peer < 0 || peer >= s->world) ? 0 : s->ch[peer].bytes.load();
}

// Bounded, ordered end: flush (limit), stop the proxy, close every channel, free the streams.
extern "C" int mesh_channels_destroy(void* h, int timeout_ms) {
  auto* s = (ChannelSet*)h;
  if (!s) return 0;
  const int halted = mesh_channels_flush(h, timeout_ms);
  s->run.store(false);
  s->cv.notify_all();
  if (s->proxy.joinable()) s->proxy.join();
  for (auto& c : s->ch) {
    for (auto& ev : c.events) cudaEventDestroy(ev.second);
    c.events.clear();
    if (c.stream != nullptr && c.state.load() != CH_HALTED) cudaStreamDestroy(c.stream);
    s->set_state(c, CH_CLOSED);
  }
  delete s;
  return halted;
}
