// HostEngine: the processor that is not a CUDA device.
//
// A placed program may put some of its layers on the host CPU (heterogeneous placement; the reference runs such
// sub-graphs on its Core ML / CPU engines over no-copy views of the shared pages, rdma/mesh-coreml.m:27-92, and
// reports which device ran each operation).  This engine executes a short list of tensor operations over host
// memory (pinned views of staging buffers, or any host pointer) on its own worker threads, asynchronously to the
// caller: submit returns a ticket, wait is bounded, and every operation's device label and wall time are
// reported.  Operations: C = A B^T (fp32 accumulate; bf16 or fp32 operands), RMSNorm, gated activation
// (SiLU or tanh-GELU of the first half times the second half), add.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

extern "C" {

enum MeshHostOpKind { MESH_HOP_GEMM_NT = 0, MESH_HOP_RMSNORM = 1, MESH_HOP_GLU = 2, MESH_HOP_ADD = 3 };
enum MeshHostDtype { MESH_HD_F32 = 0, MESH_HD_BF16 = 1 };

typedef struct MeshHostOp {
  int32_t kind, dtype;            // dtype of a, b and out (all the same)
  const void* a; const void* b; void* out;
  int64_t m, n, k;                // GEMM: out[m,n] = a[m,k] b[n,k]^T; RMSNORM/ADD: [m, n]; GLU: a[m, 2n] -> out[m, n]
  int64_t lda, ldb, ldo;
  float eps; int32_t act;         // RMSNORM: b = weight[n]; GLU: act 0 = SiLU, 1 = tanh-GELU
  double seconds;                 // filled in: wall time of this operation
  int32_t done; int32_t pad;
} MeshHostOp;

}  // extern "C"

namespace {

inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);     // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                              // round to nearest even
  return (uint16_t)(u >> 16);
}
inline float load(const void* p, int dtype, int64_t i) {
  return dtype == MESH_HD_BF16 ? bf16_to_f32(((const uint16_t*)p)[i]) : ((const float*)p)[i];
}
inline void store(void* p, int dtype, int64_t i, float v) {
  if (dtype == MESH_HD_BF16) ((uint16_t*)p)[i] = f32_to_bf16(v);
  else ((float*)p)[i] = v;
}

struct Batch {
  MeshHostOp* ops; int n; uint64_t ticket;
};

struct Engine {
  std::vector<std::thread> workers;
  std::thread driver;
  std::mutex mu;
  std::condition_variable cv, done_cv;
  std::deque<Batch> queue;
  std::atomic<bool> run{true};
  uint64_t next_ticket = 1, finished = 0;
  int threads = 1;
  // parallel-for state shared with the workers
  std::mutex pmu;
  std::condition_variable pcv, pdone;
  const MeshHostOp* cur = nullptr;
  std::atomic<int64_t> next_row{0};
  int64_t rows = 0, chunk = 1;
  int active = 0;
  uint64_t generation = 0;
};

void rows_of(const MeshHostOp& op, int64_t r0, int64_t r1) {
  const int dt = op.dtype;
  switch (op.kind) {
    case MESH_HOP_GEMM_NT: {
      std::vector<float> arow((size_t)op.k);
      for (int64_t i = r0; i < r1; ++i) {
        for (int64_t p = 0; p < op.k; ++p) arow[(size_t)p] = load(op.a, dt, i * op.lda + p);
        for (int64_t j = 0; j < op.n; ++j) {
          float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
          const int64_t base = j * op.ldb;
          int64_t p = 0;
          if (dt == MESH_HD_F32) {
            const float* b = (const float*)op.b + base;
            for (; p + 3 < op.k; p += 4) {
              acc0 += arow[p] * b[p]; acc1 += arow[p + 1] * b[p + 1];
              acc2 += arow[p + 2] * b[p + 2]; acc3 += arow[p + 3] * b[p + 3];
            }
            for (; p < op.k; ++p) acc0 += arow[p] * b[p];
          } else {
            const uint16_t* b = (const uint16_t*)op.b + base;
            for (; p + 3 < op.k; p += 4) {
              acc0 += arow[p] * bf16_to_f32(b[p]); acc1 += arow[p + 1] * bf16_to_f32(b[p + 1]);
              acc2 += arow[p + 2] * bf16_to_f32(b[p + 2]); acc3 += arow[p + 3] * bf16_to_f32(b[p + 3]);
            }
            for (; p < op.k; ++p) acc0 += arow[p] * bf16_to_f32(b[p]);
          }
          store(op.out, dt, i * op.ldo + j, (acc0 + acc1) + (acc2 + acc3));
        }
      }
      break;
    }
    case MESH_HOP_RMSNORM:
      for (int64_t i = r0; i < r1; ++i) {
        double ss = 0;
        for (int64_t j = 0; j < op.n; ++j) { float v = load(op.a, dt, i * op.lda + j); ss += (double)v * v; }
        const float r = 1.0f / std::sqrt((float)(ss / (double)op.n) + op.eps);
        for (int64_t j = 0; j < op.n; ++j)
          store(op.out, dt, i * op.ldo + j, load(op.a, dt, i * op.lda + j) * r * load(op.b, dt, j));
      }
      break;
    case MESH_HOP_GLU:
      for (int64_t i = r0; i < r1; ++i)
        for (int64_t j = 0; j < op.n; ++j) {
          const float g = load(op.a, dt, i * op.lda + j), u = load(op.a, dt, i * op.lda + op.n + j);
          float a;
          if (op.act == 0) a = g / (1.0f + std::exp(-g));
          else a = 0.5f * g * (1.0f + std::tanh(0.7978845608028654f * (g + 0.044715f * g * g * g)));
          store(op.out, dt, i * op.ldo + j, a * u);
        }
      break;
    case MESH_HOP_ADD:
      for (int64_t i = r0; i < r1; ++i)
        for (int64_t j = 0; j < op.n; ++j)
          store(op.out, dt, i * op.ldo + j, load(op.a, dt, i * op.lda + j) + load(op.b, dt, i * op.ldb + j));
      break;
    default: break;
  }
}

void worker(Engine* e) {
  uint64_t seen = 0;
  for (;;) {
    const MeshHostOp* op;
    {
      std::unique_lock<std::mutex> lk(e->pmu);
      e->pcv.wait(lk, [&] { return !e->run.load() || e->generation != seen; });
      if (!e->run.load()) return;
      seen = e->generation;
      op = e->cur;
    }
    for (;;) {
      const int64_t r0 = e->next_row.fetch_add(e->chunk);
      if (r0 >= e->rows) break;
      rows_of(*op, r0, std::min(e->rows, r0 + e->chunk));
    }
    {
      std::lock_guard<std::mutex> lk(e->pmu);
      if (--e->active == 0) e->pdone.notify_all();
    }
  }
}

void run_op(Engine* e, MeshHostOp& op) {
  const auto t0 = std::chrono::steady_clock::now();
  {
    std::unique_lock<std::mutex> lk(e->pmu);
    e->cur = &op;
    e->rows = op.m;
    e->chunk = std::max<int64_t>(1, op.m / (4 * (int64_t)e->threads));
    e->next_row.store(0);
    e->active = e->threads;
    ++e->generation;
    e->pcv.notify_all();
    e->pdone.wait(lk, [&] { return e->active == 0; });
  }
  op.seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  op.done = 1;
}

void drive(Engine* e) {
  for (;;) {
    Batch b;
    {
      std::unique_lock<std::mutex> lk(e->mu);
      e->cv.wait(lk, [&] { return !e->run.load() || !e->queue.empty(); });
      if (!e->run.load() && e->queue.empty()) return;
      b = e->queue.front();
      e->queue.pop_front();
    }
    for (int i = 0; i < b.n; ++i) run_op(e, b.ops[i]);          // operations of a batch run in order
    {
      std::lock_guard<std::mutex> lk(e->mu);
      e->finished = b.ticket;
      e->done_cv.notify_all();
    }
  }
}

}  // namespace

extern "C" {

void* mesh_host_engine_create(int threads) {
  auto* e = new Engine();
  e->threads = std::max(1, threads);
  for (int i = 0; i < e->threads; ++i) e->workers.emplace_back(worker, e);
  e->driver = std::thread(drive, e);
  return e;
}

// The operation records stay owned by the caller and must live until the ticket has been waited for.
uint64_t mesh_host_engine_submit(void* engine, MeshHostOp* ops, int n) {
  auto* e = (Engine*)engine;
  std::lock_guard<std::mutex> lk(e->mu);
  const uint64_t t = e->next_ticket++;
  for (int i = 0; i < n; ++i) { ops[i].done = 0; ops[i].seconds = 0; }
  e->queue.push_back(Batch{ops, n, t});
  e->cv.notify_all();
  return t;
}

// 0: finished; 110 (ETIMEDOUT): still running after timeout_ms.
int mesh_host_engine_wait(void* engine, uint64_t ticket, int timeout_ms) {
  auto* e = (Engine*)engine;
  std::unique_lock<std::mutex> lk(e->mu);
  const bool ok = e->done_cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return e->finished >= ticket; });
  return ok ? 0 : 110;
}

const char* mesh_host_engine_device(void*) { return "cpu"; }

void mesh_host_engine_destroy(void* engine) {
  auto* e = (Engine*)engine;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->run.store(false);
    e->cv.notify_all();
  }
  {
    std::lock_guard<std::mutex> lk(e->pmu);
    e->pcv.notify_all();
  }
  if (e->driver.joinable()) e->driver.join();
  for (auto& w : e->workers) if (w.joinable()) w.join();
  delete e;
}

}  // extern "C"
