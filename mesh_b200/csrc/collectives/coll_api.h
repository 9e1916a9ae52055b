// C ABI of the collective kernels (all-reduce, all-gather, reduce-scatter, all-to-all(v),
// broadcast, reduce, gather, scatter, send/recv, barrier) over the symmetric heap.
//
// Every collective is ONE kernel per rank with the same three steps:
//   publish  copy this rank's contribution into its own staging buffer in the symmetric heap,
//            fence at system scope and raise a counter on every peer (monotonic, never reset);
//   wait     bounded wait until the counters of the ranks it will read from reach this call's value;
//   pull     read the peers' staging buffers over NVLink (plain loads) straight into the output,
//            reducing in a fixed rank order so every rank computes bit-identical sums.
// This is the NVLink form of the reference's verbs (design/collective-verbs.md:7-35) and of its
// lowerings (rdma/mesh_compile.py:1502-1613): all-gather = each rank's part lands in place in
// the output; reduce = sum on arrival at the keeper; all-to-all(v) = per-pair blocks at their own
// sizes, never padded to the largest.
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define MESH_COLL_MAX_RANKS 8
#define MESH_COLL_HEADER_BYTES 1024     // start of each staging buffer: per-call offsets table

enum MeshDtype { MESH_F32 = 0, MESH_BF16 = 1, MESH_F16 = 2, MESH_I32 = 3, MESH_I64 = 4, MESH_U8 = 5, MESH_F64 = 6 };
enum MeshRedOp { MESH_SUM = 0, MESH_MAX = 1, MESH_MIN = 2, MESH_PROD = 3, MESH_AVG = 4 };

typedef struct MeshCommArgs {
  int rank, world;
  void* staging[MESH_COLL_MAX_RANKS];        // every rank's staging buffer of this call's parity
  uint32_t* arrived[MESH_COLL_MAX_RANKS];    // arrived[d] = rank d's counters [2][world] of this parity
  uint32_t expect_a, expect_b;               // counter values that mean "published" for step A / step B
  uint32_t add;                              // what each block adds on arrival (1); expect = calls * nblocks
  uint64_t staging_bytes;                    // capacity after the header
  void* status;
  int nblocks;
} MeshCommArgs;

int mesh_coll_max_blocks(void);
// bytes: payload of this rank.  All functions return 0 / negative argument error / positive cudaError_t.
int mesh_coll_allreduce(const MeshCommArgs* c, const void* in, void* out, uint64_t count, int dtype, int op,
                        int two_shot, void* stream);
// The same sum through the NVSwitch (multimem.ld_reduce / multimem.st on the heap's multicast mapping).
int mesh_coll_allreduce_mc(const MeshCommArgs* c, void* mc_staging, const void* in, void* out, uint64_t count, int dtype,
                           void* stream);
int mesh_coll_allgather(const MeshCommArgs* c, const void* in, void* out, uint64_t bytes_per_rank, void* stream);
// v-variant: rank r contributes counts[r] bytes placed at displs[r] in the output.
int mesh_coll_allgatherv(const MeshCommArgs* c, const void* in, void* out, const uint64_t* counts,
                         const uint64_t* displs, void* stream);
int mesh_coll_reduce_scatter(const MeshCommArgs* c, const void* in, void* out, const uint64_t* counts_elems,
                             int dtype, int op, void* stream);
// send_off/recv_off: world+1 byte offsets into in/out (block for rank j is [off[j], off[j+1])).
int mesh_coll_alltoallv(const MeshCommArgs* c, const void* in, void* out, const uint64_t* send_off,
                        const uint64_t* recv_off, void* stream);
int mesh_coll_broadcast(const MeshCommArgs* c, void* buf, uint64_t bytes, int root, void* stream);
int mesh_coll_reduce(const MeshCommArgs* c, const void* in, void* out, uint64_t count, int dtype, int op, int root,
                     void* stream);
int mesh_coll_barrier(const MeshCommArgs* c, void* stream);

// Pipelined exchange: this rank's sends (the same `in` to each listed peer) and its receive, in one launch.  A
// channel is a (source, destination) pair with a ring of `depth` pieces of `piece` bytes in the source's memory;
// `ready_base` / `ack_base` are the channel's counter totals before this message (nb arrivals per piece).
typedef struct MeshXferChan {
  void* slot;               // the ring: local for a send, on the peer for the receive
  uint32_t* ready;          // counter at the receiver
  uint32_t* ack;            // counter at the sender
  uint32_t ready_base, ack_base;
} MeshXferChan;
typedef struct MeshXferArgs {
  int n_send, has_recv, nb, depth;
  MeshXferChan send[MESH_COLL_MAX_RANKS];
  MeshXferChan recv;
  const void* in; void* out;
  uint64_t send_bytes, recv_bytes, piece;
  void* status;
} MeshXferArgs;
int mesh_p2p_exchange(const MeshXferArgs* a, void* stream);

// Test hook for the bounded-wait path: waits on a word nobody writes, with a short limit, and
// returns normally after recording TIMEOUT in the status block.
int mesh_wait_flag_test(const uint32_t* flag, uint32_t expect, uint64_t limit_ns, void* status, void* stream);

#ifdef __cplusplus
}
#endif
