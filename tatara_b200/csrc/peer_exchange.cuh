// Gradient sum over the ranks of one node by copy engines and stream memory operations (peer_exchange.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#define PX_MAX_RANKS 16
#define PX_MAX_PARTS 16
#define PX_MODE_COPY 1      // reduce-scatter and all-gather by the copy engines, a summing kernel between them
#define PX_MODE_KERNEL 2    // one kernel per part reads every rank's shard over the peer mappings and writes the sum back
#define PX_KERNEL_BLOCKS 64 // blocks of 512 threads of that kernel: enough loads in flight for the link, few SMs taken

struct PeerExchange;
// all-gathers `bytes` bytes per rank between host buffers (recv holds world * bytes); 0 on success.  Collective.
typedef int (*px_allgather_fn)(void* ctx, const void* send, void* recv, size_t bytes);

// Collective over the ranks.  arena: the base of this rank's gradient arena allocation (cudaMalloc), of which the first
// reduce_floats floats take part; loss_acc: the device double that holds this rank's loss sum.
int px_create(PeerExchange** out, int mode, int rank, int world, float* arena, size_t reduce_floats, int max_parts, double* loss_acc,
              px_allgather_fn allgather, void* allgather_ctx, std::string* err);
void px_destroy(PeerExchange* x);
// a new round of exchanges (one per training step): every rank calls it the same number of times
void px_begin_step(PeerExchange* x);
// Sum of arena[e0, e1) over the ranks, in place; the range is final on this rank when `ready` has happened.  The reduce
// kernel runs on reduce_stream; consumer_stream may read the summed range (and, with_loss, the summed loss) after the
// waits this call puts on it.  Each part index is used once per step.
int px_exchange_part(PeerExchange* x, int part, int64_t e0, int64_t e1, bool with_loss, cudaEvent_t ready,
                     cudaStream_t reduce_stream, cudaStream_t consumer_stream, int* launches, std::string* err);
// s waits until this rank's outgoing copies of the step are done: its arena may be rewritten after that
int px_join(PeerExchange* x, cudaStream_t s, std::string* err);
