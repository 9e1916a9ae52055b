// Race check of the host runtime: a driver that is compiled together with the runtime's host sources under
// ThreadSanitizer (`python -m mesh_b200._build --race-check`) and uses them the way a job does, from several threads at
// once: counters bumped while the service thread beats and while the service is stopped and started again, readers of
// the stats block, batches submitted to the host engine from two threads, the publish / poll handshake of the engine
// bridge.  Exit code 0 and no ThreadSanitizer report = no data race on these paths.  (CUDA-side ordering is checked by
// the plan checker and the bounded waits; the GPU has no such tool open on this pool.)
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <unistd.h>
#include <vector>

extern "C" {
int mesh_runtime_start(const char* group, int rank, int world, double heartbeat_s);
int mesh_runtime_stop(int unlink_block);
void mesh_runtime_count(int what, uint64_t n, int peer);
void mesh_runtime_channel(int peer, int state);
void mesh_runtime_deadline(double seconds_from_now);
int mesh_runtime_aborted(void);
void mesh_runtime_abort(int v);
int mesh_runtime_read(const char* group, int rank, uint64_t* out);

void* mesh_open(uint64_t floats);
void mesh_close(void* h);
int mesh_gather(void* h, const float* src, uint64_t offset, uint64_t count);
int mesh_scatter(void* h, float* dst, uint64_t offset, uint64_t count);
uint64_t mesh_publish(void* h);
int mesh_poll(void* h, uint64_t ticket);
float* mesh_ipc_inbox(void* h);
float* mesh_ipc_outbox(void* h);
uint64_t mesh_ipc_pending(void* h);
void mesh_ipc_complete(void* h);

typedef struct MeshHostOp {
  int32_t kind, dtype;
  const void* a; const void* b; void* out;
  int64_t m, n, k;
  int64_t lda, ldb, ldo;
  float eps; int32_t act;
  double seconds;
  int32_t done; int32_t pad;
} MeshHostOp;
void* mesh_host_engine_create(int threads);
uint64_t mesh_host_engine_submit(void* engine, MeshHostOp* ops, int n);
int mesh_host_engine_wait(void* engine, uint64_t ticket, int timeout_ms);
void mesh_host_engine_destroy(void* engine);
}

static int failures = 0;
#define EXPECT(c) do { if (!(c)) { fprintf(stderr, "race_check: %s failed (line %d)\n", #c, __LINE__); ++failures; } } while (0)

static void service_and_counters(const char* group) {
  for (int cycle = 0; cycle < 3; ++cycle) {
    EXPECT(mesh_runtime_start(group, 0, 2, 0.01) >= 0);
    std::atomic<bool> go{true};
    std::vector<std::thread> ts;
    for (int t = 0; t < 4; ++t)
      ts.emplace_back([&, t] {
        uint64_t i = 0;
        while (go.load()) {
          mesh_runtime_count(t % 3, 1, 0);
          mesh_runtime_count(3, 64, (int)(i % 8));
          mesh_runtime_count(4, i, 0);
          mesh_runtime_channel((int)(i % 8), (int)(i % 5));
          if ((i & 63) == 0) mesh_runtime_deadline(5.0);
          (void)mesh_runtime_aborted();
          ++i;
        }
      });
    ts.emplace_back([&] {
      uint64_t out[16 + 16];
      while (go.load()) {
        if (mesh_runtime_read(group, 0, out) == 0) EXPECT(out[1] == 2);
        usleep(200);
      }
    });
    usleep(30000);
    // the service goes away under the counting threads: they must fall through, not fault
    EXPECT(mesh_runtime_stop(cycle == 2) == 0);
    usleep(5000);
    go.store(false);
    for (auto& t : ts) t.join();
  }
}

static void host_engine() {
  void* e = mesh_host_engine_create(4);
  auto submitter = [&](int seed) {
    const int m = 24, n = 32, k = 40;
    std::vector<float> a(m * k), b(n * k), w(n, 1.f), c(m * n), nrm(m * n), sum(m * n);
    for (int i = 0; i < m * k; ++i) a[i] = 0.01f * (float)((i * 7 + seed) % 23 - 11);
    for (int i = 0; i < n * k; ++i) b[i] = 0.02f * (float)((i * 5 + seed) % 19 - 9);
    for (int round = 0; round < 25; ++round) {
      MeshHostOp ops[3] = {};
      ops[0].kind = 0; ops[0].a = a.data(); ops[0].b = b.data(); ops[0].out = c.data();
      ops[0].m = m; ops[0].n = n; ops[0].k = k; ops[0].lda = k; ops[0].ldb = k; ops[0].ldo = n;
      ops[1].kind = 1; ops[1].a = c.data(); ops[1].b = w.data(); ops[1].out = nrm.data();
      ops[1].m = m; ops[1].n = n; ops[1].lda = n; ops[1].ldo = n; ops[1].eps = 1e-6f;
      ops[2].kind = 3; ops[2].a = c.data(); ops[2].b = nrm.data(); ops[2].out = sum.data();
      ops[2].m = m; ops[2].n = n; ops[2].lda = n; ops[2].ldb = n; ops[2].ldo = n;
      const uint64_t t = mesh_host_engine_submit(e, ops, 3);
      EXPECT(mesh_host_engine_wait(e, t, 10000) == 0);
      EXPECT(ops[0].done && ops[1].done && ops[2].done);
      double ref = 0;
      for (int j = 0; j < k; ++j) ref += (double)a[j] * (double)b[j];
      EXPECT(std::fabs(c[0] - (float)ref) < 1e-4f);
      EXPECT(std::fabs(sum[0] - (c[0] + nrm[0])) < 1e-5f);
    }
  };
  std::thread t0(submitter, 1), t1(submitter, 2);
  t0.join();
  t1.join();
  mesh_host_engine_destroy(e);
}

static void engine_bridge() {
  void* h = mesh_open(256);
  std::atomic<bool> go{true};
  std::thread solver([&] {
    while (go.load() || mesh_ipc_pending(h)) {
      if (mesh_ipc_pending(h)) {
        const float* in = mesh_ipc_inbox(h);
        float* out = mesh_ipc_outbox(h);
        for (int i = 0; i < 256; ++i) out[i] = 2.f * in[i];
        mesh_ipc_complete(h);
      }
    }
  });
  std::vector<float> v(256), r(256);
  for (int round = 1; round <= 50; ++round) {
    for (int i = 0; i < 256; ++i) v[i] = (float)(round + i);
    EXPECT(mesh_gather(h, v.data(), 0, 256) == 0);
    const uint64_t t = mesh_publish(h);
    int spins = 0;
    while (!mesh_poll(h, t) && ++spins < 10000000) {}
    EXPECT(mesh_poll(h, t));
    EXPECT(mesh_scatter(h, r.data(), 0, 256) == 0);
    EXPECT(r[5] == 2.f * v[5]);
  }
  go.store(false);
  solver.join();
  mesh_close(h);
}

int main() {
  char group[64];
  snprintf(group, sizeof(group), "race%d", (int)getpid());
  service_and_counters(group);
  host_engine();
  engine_bridge();
  if (failures) { fprintf(stderr, "race_check: %d expectation(s) failed\n", failures); return 1; }
  printf("race_check: ok\n");
  return 0;
}
