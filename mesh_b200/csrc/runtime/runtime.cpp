// Per-process runtime service: a named shared-memory stats block (so `meshctl` and a restarted rank can
// attach to it), a low-rate service thread (heartbeat, watchdog deadline), peer-channel states, and the
// small C ABI that non-Python callers use (open / gather / scatter / publish / poll / stat).
//
// Counterparts in the reference: bridge main loop and region adoption (rdma/mesh-link.c:262-447), port
// children as a state machine (rdma/mesh-children.c:73-242), health turns (rdma/mesh-records.c:1433),
// `mesh-stat` (rdma/mesh-stat.c:65-118), and the engine bridge builtins (xonotic/darkplaces-work/mesh_ipc.c:674-704).
// On NVLink there is no NIC daemon: kernels move the data; this thread only keeps liveness and counters.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

extern "C" {

#define MESH_STATS_MAGIC 0x4d53544154533031ull      // "MSTATS01"
#define MESH_MAX_PEERS 8
enum MeshChannelState { MESH_CH_CLOSED = 0, MESH_CH_OPEN = 1, MESH_CH_MAPPED = 2, MESH_CH_CONNECTED = 3, MESH_CH_HALTED = 4 };

typedef struct MeshStats {
  uint64_t magic;
  int32_t rank, world;
  int64_t pid;
  int64_t start_ns;                 // process identity = (pid, start time), like the reference's holders
  std::atomic<uint64_t> heartbeat_ns;
  std::atomic<uint64_t> epoch;
  std::atomic<uint64_t> step;
  std::atomic<uint64_t> launches;
  std::atomic<uint64_t> collectives;
  std::atomic<uint64_t> timeouts;
  std::atomic<uint64_t> abort_flag;
  std::atomic<uint64_t> bytes_to_peer[MESH_MAX_PEERS];
  std::atomic<int32_t> channel_state[MESH_MAX_PEERS];
  std::atomic<uint64_t> deadline_ns;      // 0 = none; the service thread raises abort when it passes
  char group[64];
} MeshStats;

// Counters are bumped from any thread (launch wrappers, the channel proxy, the status monitor) without a lock, also
// while another thread stops the service: the pointer is atomic and a stopped block is never unmapped (4 KB per
// start/stop cycle stay mapped), so a reader that loaded the pointer just before a stop still writes to valid memory.
static std::atomic<MeshStats*> g_stats{nullptr};
static char g_name[128];
static std::thread g_thread;
static std::atomic<bool> g_run{false};
static std::mutex g_mu;

static uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

static MeshStats* map_block(const char* name, int create) {
  int fd = shm_open(name, create ? (O_RDWR | O_CREAT) : O_RDONLY, 0644);
  if (fd < 0) return nullptr;
  if (create && ftruncate(fd, sizeof(MeshStats)) != 0) { close(fd); return nullptr; }
  void* p = mmap(nullptr, sizeof(MeshStats), create ? (PROT_READ | PROT_WRITE) : PROT_READ, MAP_SHARED, fd, 0);
  close(fd);
  return p == MAP_FAILED ? nullptr : (MeshStats*)p;
}

// Create (or re-adopt after a restart) this rank's stats block and start the service thread.
int mesh_runtime_stop(int unlink_block);
int mesh_runtime_start(const char* group, int rank, int world, double heartbeat_s) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_stats.load()) return 0;
  snprintf(g_name, sizeof(g_name), "/mesh_b200_%s_%d", group, rank);
  MeshStats* s = map_block(g_name, 1);
  if (!s) return -1;
  const bool adopt = s->magic == MESH_STATS_MAGIC && s->rank == rank && s->world == world;
  if (!adopt) memset((void*)s, 0, sizeof(*s));
  s->magic = MESH_STATS_MAGIC;
  s->rank = rank; s->world = world;
  s->pid = (int64_t)getpid();
  s->start_ns = (int64_t)now_ns();
  snprintf(s->group, sizeof(s->group), "%s", group);
  s->heartbeat_ns.store(now_ns());
  s->abort_flag.store(0);
  g_stats.store(s);
  g_run.store(true);
  static bool at_exit_installed = false;
  if (!at_exit_installed) {
    // a process that ends without calling stop (an exception on its way out) still joins the service thread before the
    // thread object is destroyed; the block stays for a supervisor to read
    at_exit_installed = true;
    atexit([] { mesh_runtime_stop(0); });
  }
  const auto period = std::chrono::milliseconds((int)(heartbeat_s > 0.01 ? heartbeat_s * 1000 : 10));
  g_thread = std::thread([period, s] {
    while (g_run.load()) {
      s->heartbeat_ns.store(now_ns());
      const uint64_t dl = s->deadline_ns.load();
      if (dl && now_ns() > dl) s->abort_flag.store(1);
      // sleep in short slices so that a stop request is honoured within milliseconds, not a heartbeat period
      for (auto left = period; left.count() > 0 && g_run.load(); left -= std::chrono::milliseconds(20))
        std::this_thread::sleep_for(std::min<std::chrono::milliseconds>(left, std::chrono::milliseconds(20)));
    }
  });
  return adopt ? 1 : 0;
}

// Bounded, ordered stop: the thread is joined, channels are marked closed, the block stays for readers
// unless `unlink` is set.
int mesh_runtime_stop(int unlink_block) {
  std::lock_guard<std::mutex> lk(g_mu);
  MeshStats* s = g_stats.load();
  if (!s) return 0;
  g_run.store(false);
  if (g_thread.joinable()) g_thread.join();
  g_stats.store(nullptr);
  for (int i = 0; i < MESH_MAX_PEERS; ++i) s->channel_state[i].store(MESH_CH_CLOSED);
  s->heartbeat_ns.store(0);
  if (unlink_block) shm_unlink(g_name);
  return 0;
}

void mesh_runtime_count(int what, uint64_t n, int peer) {
  MeshStats* s = g_stats.load();
  if (!s) return;
  switch (what) {
    case 0: s->launches.fetch_add(n); break;
    case 1: s->collectives.fetch_add(n); break;
    case 2: s->timeouts.fetch_add(n); break;
    case 3: if (peer >= 0 && peer < MESH_MAX_PEERS) s->bytes_to_peer[peer].fetch_add(n); break;
    case 4: s->step.store(n); break;
    case 5: s->epoch.store(n); break;
  }
}
void mesh_runtime_channel(int peer, int state) {
  MeshStats* s = g_stats.load();
  if (s && peer >= 0 && peer < MESH_MAX_PEERS) s->channel_state[peer].store(state);
}
void mesh_runtime_deadline(double seconds_from_now) {
  MeshStats* s = g_stats.load();
  if (s) s->deadline_ns.store(seconds_from_now > 0 ? now_ns() + (uint64_t)(seconds_from_now * 1e9) : 0);
}
int mesh_runtime_aborted(void) { MeshStats* s = g_stats.load(); return s ? (int)s->abort_flag.load() : 0; }
void mesh_runtime_abort(int v) { MeshStats* s = g_stats.load(); if (s) s->abort_flag.store((uint64_t)v); }

// Read-only view of any rank's block (what `meshctl status` prints).  Returns 0, or -1 when absent.
int mesh_runtime_read(const char* group, int rank, uint64_t* out /*[16 + 2*MESH_MAX_PEERS]*/) {
  char name[128];
  snprintf(name, sizeof(name), "/mesh_b200_%s_%d", group, rank);
  MeshStats* s = map_block(name, 0);
  if (!s) return -1;
  int rc = 0;
  if (s->magic != MESH_STATS_MAGIC) rc = -2;
  else {
    out[0] = (uint64_t)s->rank; out[1] = (uint64_t)s->world; out[2] = (uint64_t)s->pid; out[3] = (uint64_t)s->start_ns;
    out[4] = s->heartbeat_ns.load(); out[5] = s->epoch.load(); out[6] = s->step.load(); out[7] = s->launches.load();
    out[8] = s->collectives.load(); out[9] = s->timeouts.load(); out[10] = s->abort_flag.load(); out[11] = now_ns();
    for (int i = 0; i < MESH_MAX_PEERS; ++i) {
      out[16 + i] = s->bytes_to_peer[i].load();
      out[16 + MESH_MAX_PEERS + i] = (uint64_t)s->channel_state[i].load();
    }
  }
  munmap((void*)s, sizeof(MeshStats));
  return rc;
}

// ---- the engine-bridge shaped C ABI (host buffers; non-blocking publish + poll)
typedef struct MeshIpc { float* inbox; float* outbox; uint64_t n; std::atomic<uint64_t> published, consumed; } MeshIpc;

void* mesh_open(uint64_t floats) {
  MeshIpc* h = new MeshIpc();
  h->inbox = new float[floats]();
  h->outbox = new float[floats]();
  h->n = floats;
  h->published.store(0);
  h->consumed.store(0);
  return h;
}
void mesh_close(void* hv) {
  MeshIpc* h = (MeshIpc*)hv;
  if (!h) return;
  delete[] h->inbox;
  delete[] h->outbox;
  delete h;
}
// gather: caller's values -> the inbox at an offset; scatter: the outbox -> caller's buffer
int mesh_gather(void* hv, const float* src, uint64_t offset, uint64_t count) {
  MeshIpc* h = (MeshIpc*)hv;
  if (!h || offset + count > h->n) return -1;
  memcpy(h->inbox + offset, src, count * sizeof(float));
  return 0;
}
int mesh_scatter(void* hv, float* dst, uint64_t offset, uint64_t count) {
  MeshIpc* h = (MeshIpc*)hv;
  if (!h || offset + count > h->n) return -1;
  memcpy(dst, h->outbox + offset, count * sizeof(float));
  return 0;
}
uint64_t mesh_publish(void* hv) { return ((MeshIpc*)hv)->published.fetch_add(1) + 1; }       // returns the ticket
int mesh_poll(void* hv, uint64_t ticket) { return ((MeshIpc*)hv)->consumed.load() >= ticket ? 1 : 0; }
// the solver side: take the inbox, leave results in the outbox, mark tickets consumed
float* mesh_ipc_inbox(void* hv) { return ((MeshIpc*)hv)->inbox; }
float* mesh_ipc_outbox(void* hv) { return ((MeshIpc*)hv)->outbox; }
uint64_t mesh_ipc_pending(void* hv) { MeshIpc* h = (MeshIpc*)hv; return h->published.load() - h->consumed.load(); }
void mesh_ipc_complete(void* hv) { MeshIpc* h = (MeshIpc*)hv; h->consumed.store(h->published.load()); }
int mesh_stat(void* hv, uint64_t* out3) {
  MeshIpc* h = (MeshIpc*)hv;
  if (!h) return -1;
  out3[0] = h->n; out3[1] = h->published.load(); out3[2] = h->consumed.load();
  return 0;
}

}  // extern "C"
