// Gradient sum over the data-parallel ranks of one node without a kernel that holds SMs for the transfer.
//
// The all-reduce of a range of the gradient arena is a reduce-scatter followed by an all-gather, both done by the copy
// engines over NVLink peer mappings (cudaMemcpyAsync between this rank's memory and the peers' memory opened through
// CUDA IPC), with stream memory operations as the signals between ranks:
//   A  push     rank r copies shard q of its range into rank q's receive window, for every q != r, then writes the step's
//               sequence number into q's flag "r has pushed part p";
//   B  reduce   r waits (cuStreamWaitValue32, no kernel spins) for every peer's push flag and sums its own shard over the
//               ranks in rank order 0, 1, .. (one small kernel, bitwise the same on every run);
//   C  publish  r copies the reduced shard into every peer's arena and writes q's flag "r has published part p";
//   D  consume  the consumer stream waits for every peer's publish flag: the whole range is then the sum on every rank,
//               the same bits everywhere because each element was summed by exactly one rank.
// The FT weight gradient kernel holds every SM (one 1024-thread block with 208 KB of shared memory each); NCCL's ring
// kernels wait for SMs beside it and slow it down, the copy engines do neither.
//
// Buffers are reused from step to step without further signals: a peer starts step s + 1 only after it has seen this
// rank's publish flags of step s, which are written behind this rank's reduce of step s (stream order), so the receive
// windows are free when the peer's next push arrives; arena ranges are overwritten by a peer's publish only after this
// rank's push of the same part has been flagged to that peer.  Flags carry a sequence number that only grows.
//
// Second form (PX_MODE_KERNEL): the same signals, but the data moves in one kernel per part and rank: rank r reads shard r of
// every rank's arena through the peer mappings (NVLink loads), sums in rank order and stores the sum into shard r of every
// rank's arena (NVLink stores): no receive windows, no copy engines, a few SMs taken for the time of the transfer.
// Measured (config 3, fp32, ms per step): two B200s copy form 4.69, NCCL 4.82; four B200s copy form 4.98, NCCL 5.00, kernel
// form 5.17.  Between two idle GPUs a 23 MB peer copy runs at 640 GB/s per direction; inside the step, next to the gradient
// kernel and with pushes and publishes of neighbouring parts sharing the links, a part's 69 MB took 0.25 to 0.3 ms.
//
// A rank that dies leaves its peers' streams waiting: there is no time-out on a stream wait.  The host notices through
// the loss read-back of tb_train_step (a deadline) and the handle is poisoned; the process has to end to free the GPU
// queue.  No wait here is a spinning kernel.
#include "common.cuh"
#include "peer_exchange.cuh"

#include <stdio.h>
#include <string.h>

#include <vector>

namespace {

struct SrcList {
    const float* p[PX_MAX_RANKS];
};

__global__ void __launch_bounds__(256) k_px_reduce(float4* dst, SrcList src, int world, size_t n4) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 a = __ldcg(reinterpret_cast<const float4*>(src.p[0]) + i);
        for (int q = 1; q < world; ++q) {
            const float4 b = __ldcg(reinterpret_cast<const float4*>(src.p[q]) + i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        dst[i] = a;
    }
}

struct BufList {
    float* p[PX_MAX_RANKS];
};

// every rank's shard (bufs.p[q] = rank q's arena at this rank's shard) summed in rank order and written back to all of them
__global__ void __launch_bounds__(512) k_px_allreduce(BufList bufs, int world, size_t n4) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += 2 * stride) {
        const size_t j = i + stride;
        const bool two = j < n4;
        float4 a = __ldcg(reinterpret_cast<const float4*>(bufs.p[0]) + i);
        float4 b = two ? __ldcg(reinterpret_cast<const float4*>(bufs.p[0]) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 1; q < world; ++q) {
            const float4 u = __ldcg(reinterpret_cast<const float4*>(bufs.p[q]) + i);
            const float4 v = two ? __ldcg(reinterpret_cast<const float4*>(bufs.p[q]) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
            b.x += v.x; b.y += v.y; b.z += v.z; b.w += v.w;
        }
        for (int q = 0; q < world; ++q) {
            __stcg(reinterpret_cast<float4*>(bufs.p[q]) + i, a);
            if (two) __stcg(reinterpret_cast<float4*>(bufs.p[q]) + j, b);
        }
    }
}

struct LossList {
    const double* p[PX_MAX_RANKS];
};

__global__ void k_px_loss(double* __restrict__ dst, LossList src, int world) {
    double a = src.p[0][0];
    for (int q = 1; q < world; ++q) a += src.p[q][0];
    *dst = a;
}

typedef int (*StreamValue32Fn)(cudaStream_t, unsigned long long, unsigned, unsigned);

}  // namespace

struct PeerExchange {
    int mode = PX_MODE_COPY;
    int world = 0, rank = 0, max_parts = 0;
    size_t reduce_floats = 0;
    float* arena = nullptr;
    double* loss_acc = nullptr;
    unsigned char* block = nullptr;  // this rank's flags, loss slots and receive windows (one allocation, one IPC handle)
    size_t off_loss = 0, off_recv = 0;
    float* peer_arena[PX_MAX_RANKS] = {};
    unsigned char* peer_block[PX_MAX_RANKS] = {};
    bool opened_arena[PX_MAX_RANKS] = {}, opened_block[PX_MAX_RANKS] = {};
    cudaStream_t push_stream = nullptr, publish_stream = nullptr;  // join points of the per-peer copy streams
    // a stream per peer and direction, so that copies to different peers need not queue behind one another
    cudaStream_t peer_push[PX_MAX_RANKS] = {}, peer_publish[PX_MAX_RANKS] = {};
    cudaEvent_t ev_peer_push[PX_MAX_RANKS] = {}, ev_peer_publish[PX_MAX_RANKS] = {}, ev_loss_slot = nullptr;
    cudaEvent_t ev_reduced[PX_MAX_PARTS] = {}, ev_push_done = nullptr, ev_publish_done = nullptr;
    unsigned seq = 0;
    StreamValue32Fn wait_value = nullptr, write_value = nullptr;

    // flags: [kind 0 pushed / 1 published][sender][part]
    size_t flag_off(int kind, int sender, int part) const { return (((size_t)kind * PX_MAX_RANKS + sender) * PX_MAX_PARTS + part) * 4; }
    float* recv_window(unsigned char* blk, int sender) const { return reinterpret_cast<float*>(blk + off_recv) + (size_t)sender * reduce_floats; }
};

#define PXC(call)                                                                                  \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            if (err) *err = std::string(#call) + ": " + cudaGetErrorString(e_);                    \
            return -1;                                                                             \
        }                                                                                          \
    } while (0)

void px_destroy(PeerExchange* x) {
    if (!x) return;
    for (int q = 0; q < x->world; ++q) {
        if (x->opened_arena[q]) cudaIpcCloseMemHandle(x->peer_arena[q]);
        if (x->opened_block[q]) cudaIpcCloseMemHandle(x->peer_block[q]);
    }
    if (x->push_stream) cudaStreamDestroy(x->push_stream);
    if (x->publish_stream) cudaStreamDestroy(x->publish_stream);
    for (auto& st : x->peer_push) if (st) cudaStreamDestroy(st);
    for (auto& st : x->peer_publish) if (st) cudaStreamDestroy(st);
    for (auto& e : x->ev_peer_push) if (e) cudaEventDestroy(e);
    for (auto& e : x->ev_peer_publish) if (e) cudaEventDestroy(e);
    if (x->ev_loss_slot) cudaEventDestroy(x->ev_loss_slot);
    for (auto& e : x->ev_reduced) if (e) cudaEventDestroy(e);
    if (x->ev_push_done) cudaEventDestroy(x->ev_push_done);
    if (x->ev_publish_done) cudaEventDestroy(x->ev_publish_done);
    cudaFree(x->block);
    delete x;
}

int px_create(PeerExchange** out, int mode, int rank, int world, float* arena, size_t reduce_floats, int max_parts, double* loss_acc,
              px_allgather_fn allgather, void* allgather_ctx, std::string* err) {
    *out = nullptr;
    if (world < 2 || world > PX_MAX_RANKS || max_parts > PX_MAX_PARTS || reduce_floats % 4 != 0) {
        if (err) *err = "peer exchange: 2.." + std::to_string(PX_MAX_RANKS) + " ranks of one node, range a multiple of 4 floats";
        return -1;
    }
    PeerExchange* x = new PeerExchange;
    x->mode = mode; x->world = world; x->rank = rank; x->max_parts = max_parts; x->reduce_floats = reduce_floats; x->arena = arena; x->loss_acc = loss_acc;
    struct Guard { PeerExchange* x; bool keep = false; ~Guard() { if (!keep) px_destroy(x); } } guard{x};
    // every rank's two IPC handles; ok = 0 tells the others that this rank could not get that far
    struct Card { cudaIpcMemHandle_t arena, block; int ok; int pad[3]; };
    std::vector<Card> cards(world);
    Card mine;
    memset(&mine, 0, sizeof mine);
    // Both all-gathers below are reached by every rank whatever failed locally, and every rank leaves with the same
    // verdict: a rank that gave up alone would leave the others waiting in a collective.
    auto local_setup = [&]() -> int {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult st;
        PXC(cudaGetDriverEntryPoint("cuStreamWaitValue32", &fn, cudaEnableDefault, &st));
        if (st != cudaDriverEntryPointSuccess || !fn) { if (err) *err = "cuStreamWaitValue32 is not available in this driver"; return -1; }
        x->wait_value = (StreamValue32Fn)fn;
        PXC(cudaGetDriverEntryPoint("cuStreamWriteValue32", &fn, cudaEnableDefault, &st));
        if (st != cudaDriverEntryPointSuccess || !fn) { if (err) *err = "cuStreamWriteValue32 is not available in this driver"; return -1; }
        x->write_value = (StreamValue32Fn)fn;
        const size_t flag_bytes = (size_t)2 * PX_MAX_RANKS * PX_MAX_PARTS * 4;
        x->off_loss = (flag_bytes + 255) / 256 * 256;
        x->off_recv = x->off_loss + (PX_MAX_RANKS * sizeof(double) + 255) / 256 * 256;
        const size_t block_bytes = x->off_recv + (mode == PX_MODE_COPY ? (size_t)world * reduce_floats * 4 : 0);  // receive windows
        PXC(cudaMalloc((void**)&x->block, block_bytes));
        PXC(cudaMemset(x->block, 0, x->off_recv));  // flags (sequence 0 = nothing yet) and loss slots
        PXC(cudaDeviceSynchronize());
        PXC(cudaIpcGetMemHandle(&mine.arena, arena));
        PXC(cudaIpcGetMemHandle(&mine.block, x->block));
        int lo = 0, hi = 0;
        PXC(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        PXC(cudaStreamCreateWithPriority(&x->push_stream, cudaStreamNonBlocking, hi));
        PXC(cudaStreamCreateWithPriority(&x->publish_stream, cudaStreamNonBlocking, hi));
        for (int q = 0; q < world; ++q) {
            if (q == rank) continue;
            PXC(cudaStreamCreateWithPriority(&x->peer_push[q], cudaStreamNonBlocking, hi));
            PXC(cudaStreamCreateWithPriority(&x->peer_publish[q], cudaStreamNonBlocking, hi));
            PXC(cudaEventCreateWithFlags(&x->ev_peer_push[q], cudaEventDisableTiming));
            PXC(cudaEventCreateWithFlags(&x->ev_peer_publish[q], cudaEventDisableTiming));
        }
        PXC(cudaEventCreateWithFlags(&x->ev_loss_slot, cudaEventDisableTiming));
        for (int p = 0; p < max_parts; ++p) PXC(cudaEventCreateWithFlags(&x->ev_reduced[p], cudaEventDisableTiming));
        PXC(cudaEventCreateWithFlags(&x->ev_push_done, cudaEventDisableTiming));
        PXC(cudaEventCreateWithFlags(&x->ev_publish_done, cudaEventDisableTiming));
        return 0;
    };
    mine.ok = local_setup() == 0 ? 1 : 0;
    if (allgather(allgather_ctx, &mine, cards.data(), sizeof(Card)) != 0) { if (err) *err = "peer exchange: handle all-gather failed"; return -1; }
    auto open_peers = [&]() -> int {
        for (int q = 0; q < world; ++q)
            if (!cards[q].ok) { if (err && q != rank) *err = "peer exchange: rank " + std::to_string(q) + " could not set up its buffers"; return -1; }
        for (int q = 0; q < world; ++q) {
            if (q == rank) { x->peer_arena[q] = arena; x->peer_block[q] = x->block; continue; }
            PXC(cudaIpcOpenMemHandle((void**)&x->peer_arena[q], cards[q].arena, cudaIpcMemLazyEnablePeerAccess));
            x->opened_arena[q] = true;
            PXC(cudaIpcOpenMemHandle((void**)&x->peer_block[q], cards[q].block, cudaIpcMemLazyEnablePeerAccess));
            x->opened_block[q] = true;
        }
        return 0;
    };
    struct Verdict { int ok; int pad[3]; } v{open_peers() == 0 ? 1 : 0, {0, 0, 0}};
    std::vector<Verdict> all(world);
    if (allgather(allgather_ctx, &v, all.data(), sizeof(Verdict)) != 0) { if (err) *err = "peer exchange: verdict all-gather failed"; return -1; }
    for (int q = 0; q < world; ++q)
        if (!all[q].ok) {
            if (err && q != rank) *err = "peer exchange: rank " + std::to_string(q) + " could not map its peers' memory";
            return -1;
        }
    guard.keep = true;
    *out = x;
    return 0;
}

void px_begin_step(PeerExchange* x) { x->seq += 1; }

// shard boundaries of [e0, e1): equal shares in units of 4 floats (e0 and e1 are multiples of 4)
static inline int64_t shard_bound(int64_t e0, int64_t e1, int q, int world) { return e0 + ((e1 - e0) / 4 * q / world) * 4; }

int px_exchange_part(PeerExchange* x, int part, int64_t e0, int64_t e1, bool with_loss, cudaEvent_t ready,
                     cudaStream_t reduce_stream, cudaStream_t consumer_stream, int* launches, std::string* err) {
    const int G = x->world, r = x->rank;
    if (part < 0 || part >= x->max_parts || e0 % 4 != 0 || e1 % 4 != 0 || e1 < e0 || (size_t)e1 > x->reduce_floats) {
        if (err) *err = "peer exchange: bad part";
        return -1;
    }
#define PXD(call)                                                                                  \
    do {                                                                                           \
        int e_ = (call);                                                                           \
        if (e_ != 0) {                                                                             \
            if (err) *err = std::string(#call) + ": driver error " + std::to_string(e_);          \
            return -1;                                                                             \
        }                                                                                          \
    } while (0)
    if (x->mode == PX_MODE_KERNEL) {
        unsigned char* my_slot = x->block + x->off_loss + (size_t)r * sizeof(double);
        // A  this rank's range (and loss slot) is final: tell the peers
        PXC(cudaStreamWaitEvent(x->push_stream, ready, 0));
        if (with_loss) {
            PXC(cudaMemcpyAsync(my_slot, x->loss_acc, sizeof(double), cudaMemcpyDeviceToDevice, x->push_stream));
            PXC(cudaEventRecord(x->ev_loss_slot, x->push_stream));
        }
        for (int i = 1; i < G; ++i) {
            const int q = (r + i) % G;
            PXD(x->write_value(x->push_stream, (unsigned long long)(uintptr_t)(x->peer_block[q] + x->flag_off(0, r, part)), x->seq, 0));
        }
        PXC(cudaEventRecord(x->ev_push_done, x->push_stream));
        // B  when every rank's range is final: this rank's shard, summed in rank order, into every rank's arena
        PXC(cudaStreamWaitEvent(reduce_stream, ready, 0));
        for (int q = 0; q < G; ++q)
            if (q != r) PXD(x->wait_value(reduce_stream, (unsigned long long)(uintptr_t)(x->block + x->flag_off(0, q, part)), x->seq, 0));
        const int64_t k0 = shard_bound(e0, e1, r, G), k1 = shard_bound(e0, e1, r + 1, G);
        if (k1 > k0) {
            BufList bufs;
            for (int q = 0; q < G; ++q) bufs.p[q] = x->peer_arena[q] + k0;
            const size_t n4 = (size_t)(k1 - k0) / 4;
            const int blocks = (int)((n4 + 1023) / 1024 < PX_KERNEL_BLOCKS ? (n4 + 1023) / 1024 : PX_KERNEL_BLOCKS);
            k_px_allreduce<<<blocks, 512, 0, reduce_stream>>>(bufs, G, n4);
            *launches += 1;
        }
        if (with_loss) {
            PXC(cudaStreamWaitEvent(reduce_stream, x->ev_loss_slot, 0));
            LossList src;  // every rank's own slot, read where it lies
            for (int q = 0; q < G; ++q) src.p[q] = reinterpret_cast<const double*>(x->peer_block[q] + x->off_loss) + q;
            k_px_loss<<<1, 1, 0, reduce_stream>>>(x->loss_acc, src, G);
            *launches += 1;
        }
        PXC(cudaGetLastError());
        PXC(cudaEventRecord(x->ev_reduced[part], reduce_stream));
        // C  tell the peers that shard r of the part is the sum
        PXC(cudaStreamWaitEvent(x->publish_stream, x->ev_reduced[part], 0));
        for (int i = 1; i < G; ++i) {
            const int q = (r + i) % G;
            PXD(x->write_value(x->publish_stream, (unsigned long long)(uintptr_t)(x->peer_block[q] + x->flag_off(1, r, part)), x->seq, 0));
        }
        PXC(cudaEventRecord(x->ev_publish_done, x->publish_stream));
        // D  the consumer sees the whole range summed
        PXC(cudaStreamWaitEvent(consumer_stream, x->ev_reduced[part], 0));
        for (int q = 0; q < G; ++q)
            if (q != r) PXD(x->wait_value(consumer_stream, (unsigned long long)(uintptr_t)(x->block + x->flag_off(1, q, part)), x->seq, 0));
        return 0;
    }
    // A  push (a stream per peer)
    // (the loss goes through this rank's own slot: loss_acc itself is overwritten by the sum in step B)
    unsigned char* my_loss = x->block + x->off_loss + (size_t)r * sizeof(double);
    if (with_loss) {
        PXC(cudaStreamWaitEvent(x->push_stream, ready, 0));
        PXC(cudaMemcpyAsync(my_loss, x->loss_acc, sizeof(double), cudaMemcpyDeviceToDevice, x->push_stream));
        PXC(cudaEventRecord(x->ev_loss_slot, x->push_stream));
    }
    for (int i = 1; i < G; ++i) {
        const int q = (r + i) % G;
        cudaStream_t sq = x->peer_push[q];
        PXC(cudaStreamWaitEvent(sq, ready, 0));
        const int64_t b0 = shard_bound(e0, e1, q, G), b1 = shard_bound(e0, e1, q + 1, G);
        if (b1 > b0)
            PXC(cudaMemcpyAsync(x->recv_window(x->peer_block[q], r) + b0, x->arena + b0, (size_t)(b1 - b0) * 4, cudaMemcpyDefault, sq));
        if (with_loss) {
            PXC(cudaStreamWaitEvent(sq, x->ev_loss_slot, 0));
            PXC(cudaMemcpyAsync(x->peer_block[q] + x->off_loss + (size_t)r * sizeof(double), my_loss, sizeof(double), cudaMemcpyDefault, sq));
        }
        PXD(x->write_value(sq, (unsigned long long)(uintptr_t)(x->peer_block[q] + x->flag_off(0, r, part)), x->seq, 0));
        PXC(cudaEventRecord(x->ev_peer_push[q], sq));
        PXC(cudaStreamWaitEvent(x->push_stream, x->ev_peer_push[q], 0));
    }
    PXC(cudaEventRecord(x->ev_push_done, x->push_stream));
    // B  reduce this rank's shard in rank order
    PXC(cudaStreamWaitEvent(reduce_stream, ready, 0));
    for (int q = 0; q < G; ++q)
        if (q != r) PXD(x->wait_value(reduce_stream, (unsigned long long)(uintptr_t)(x->block + x->flag_off(0, q, part)), x->seq, /*CU_STREAM_WAIT_VALUE_GEQ*/ 0));
    const int64_t m0 = shard_bound(e0, e1, r, G), m1 = shard_bound(e0, e1, r + 1, G);
    if (m1 > m0) {
        SrcList src;
        for (int q = 0; q < G; ++q) src.p[q] = q == r ? x->arena + m0 : x->recv_window(x->block, q) + m0;
        const size_t n4 = (size_t)(m1 - m0) / 4;
        const int blocks = (int)((n4 + 255) / 256 < 148 * 4 ? (n4 + 255) / 256 : 148 * 4);
        k_px_reduce<<<blocks, 256, 0, reduce_stream>>>(reinterpret_cast<float4*>(x->arena + m0), src, G, n4);
        *launches += 1;
    }
    if (with_loss) {
        // this rank's own slot is written on the push stream
        PXC(cudaStreamWaitEvent(reduce_stream, x->ev_loss_slot, 0));
        LossList src;
        for (int q = 0; q < G; ++q) src.p[q] = reinterpret_cast<const double*>(x->block + x->off_loss) + q;
        k_px_loss<<<1, 1, 0, reduce_stream>>>(x->loss_acc, src, G);
        *launches += 1;
    }
    PXC(cudaGetLastError());
    PXC(cudaEventRecord(x->ev_reduced[part], reduce_stream));
    // C  publish the reduced shard (a stream per peer)
    for (int i = 1; i < G; ++i) {
        const int q = (r + i) % G;
        cudaStream_t sq = x->peer_publish[q];
        PXC(cudaStreamWaitEvent(sq, x->ev_reduced[part], 0));
        if (m1 > m0)
            PXC(cudaMemcpyAsync(x->peer_arena[q] + m0, x->arena + m0, (size_t)(m1 - m0) * 4, cudaMemcpyDefault, sq));
        PXD(x->write_value(sq, (unsigned long long)(uintptr_t)(x->peer_block[q] + x->flag_off(1, r, part)), x->seq, 0));
        PXC(cudaEventRecord(x->ev_peer_publish[q], sq));
        PXC(cudaStreamWaitEvent(x->publish_stream, x->ev_peer_publish[q], 0));
    }
    PXC(cudaEventRecord(x->ev_publish_done, x->publish_stream));
    // D  the consumer sees the whole range summed
    PXC(cudaStreamWaitEvent(consumer_stream, x->ev_reduced[part], 0));
    for (int q = 0; q < G; ++q)
        if (q != r) PXD(x->wait_value(consumer_stream, (unsigned long long)(uintptr_t)(x->block + x->flag_off(1, q, part)), x->seq, 0));
    return 0;
#undef PXD
}

// s waits until this rank's outgoing copies of the step have left its arena (the arena may then be rewritten)
int px_join(PeerExchange* x, cudaStream_t s, std::string* err) {
    PXC(cudaStreamWaitEvent(s, x->ev_push_done, 0));
    PXC(cudaStreamWaitEvent(s, x->ev_publish_done, 0));
    return 0;
}
