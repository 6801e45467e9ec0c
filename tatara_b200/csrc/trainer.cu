// The trainer behind the C ABI: owns the parameter groups, the workspace, the input and loss rings and
// drives one training step as a fixed sequence of kernels on one compute stream (inputs arrive on a
// copy stream).  Mirrors GpuTrainer (bins/nnue_train/src/trainer_layerstack.rs) and SimpleGpuTrainer
// (bins/nnue_train/src/trainer_simple.rs) at the level of the TrainerBackend trait.
#include "common.cuh"
#include "peer_exchange.cuh"
#include "../../include/tatara_b200.h"

#include <cuda_fp16.h>
#include <dlfcn.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <climits>
#include <string>
#include <thread>
#include <vector>

#define FT_POST_SCALE (127.0f / 128.0f)  // bins/nnue_train/src/arch.rs:64-70
#define CLAMP_Q (127.0f / 64.0f)         // arch.rs:138-143: i8::MAX / QB
#define CLAMP_NONE 3.402823466e+38f      // arch.rs:145-148: f32::MAX sentinel
#define BETA2 0.999f                     // crates/nnue-train/src/optimizer.rs:122-130 RangerParams::DEFAULT
#define EPS 1e-8f
#define RANGER_ALPHA 0.5f
#define RANGER_K 6
#define N_SMA_THRESHOLD 5.0f
#define FT_DFT_FP16_BASE_SCALE 16384.0f  // arch.rs:72-93: the fp16 dft rows carry gradient * 2^14 * batch
#define DGRAD_CTAS (148 * 2)
#define AR_PARTS_MAX 6
#define PEER_DEADLINE_S 120  // peer exchange: longest wait for a step before the peers are given up
// Number of launches the FT weight gradient is cut into in data-parallel runs (each part's all-reduce and row updates
// overlap the next part).  A part runs slices x strips blocks of one per SM: the count that wastes the fewest block
// slots wins, a shorter last part (whose communication nothing hides) breaking near ties.  Measured on two B200s at
// 45 slices x 48 strips (peer exchange, row updates at low priority): 5 parts 4.70 ms per step, 3 parts 4.78, 4 parts 4.87,
// 6 parts 4.87, 9 parts 4.91; unequal parts with a short last one 4.67 at best.
static int ar_parts_for(int n_slices, int strips, int n_sm) {
    int best = 1;
    double best_cost = 1e30;
    for (int parts = 3; parts <= AR_PARTS_MAX; ++parts) {
        if (n_slices < 2 * parts) break;
        double waves = 0, last = 0;
        for (int p = 0; p < parts; ++p) {
            const int k0 = (int)((int64_t)n_slices * p / parts), k1 = (int)((int64_t)n_slices * (p + 1) / parts);
            last = (double)(((k1 - k0) * strips + n_sm - 1) / n_sm);
            waves += last;
        }
        const double cost = waves + 0.35 * last;
        if (cost < best_cost) { best_cost = cost; best = parts; }
    }
    return best;
}

namespace {

thread_local std::string g_create_error;

// ---- NCCL through dlopen: the library has no link-time dependency on it -----------------------------
struct Uid { char internal[128]; };  // ncclUniqueId
struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(void*) = nullptr;
    int (*CommInitRank)(void**, int, Uid, int) = nullptr;
    int (*CommInitRankConfig)(void**, int, Uid, int, void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
};
NcclApi g_nccl;

bool load_nccl(std::string* err) {
    if (g_nccl.lib) return true;
    // NCCL's environment belongs to the application: nothing is set here.  (The all-reduces of this library run next to
    // kernels that hold every SM; on eight B200s, 460 MB in five parts behind the FT weight gradient, a step measured 5.32 ms
    // with NCCL's NVLS algorithm and 5.11 ms with NCCL_NVLS_ENABLE=0, so the benchmark sets that, and a fixed NCCL_ALGO /
    // NCCL_PROTO, itself.)
    const char* names[] = {getenv("TATARA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n || !*n) continue;
        g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.lib) break;
    }
    if (!g_nccl.lib) { *err = "cannot load libnccl.so.2 (set TATARA_NCCL_LIB to its path)"; return false; }
#define SYM(field, name) *(void**)(&g_nccl.field) = dlsym(g_nccl.lib, name); if (!g_nccl.field) { *err = std::string("missing symbol ") + name; g_nccl.lib = nullptr; return false; }
    SYM(GetUniqueId, "ncclGetUniqueId")
    SYM(CommInitRank, "ncclCommInitRank")
    SYM(CommInitRankConfig, "ncclCommInitRankConfig")
    SYM(AllReduce, "ncclAllReduce")
    SYM(AllGather, "ncclAllGather")
    SYM(CommDestroy, "ncclCommDestroy")
    SYM(GetErrorString, "ncclGetErrorString")
    SYM(GroupStart, "ncclGroupStart")
    SYM(GroupEnd, "ncclGroupEnd")
#undef SYM
    return true;
}

struct Group {
    std::string name;
    int kind;  // 0 ft, 1 dense, 2 bias
    float clamp;
    int64_t len;
    float *w = nullptr, *m = nullptr, *v = nullptr, *slow = nullptr, *grad = nullptr;
};

struct DevBatch {
    int *stm = nullptr, *nstm = nullptr, *nnz = nullptr, *bucket = nullptr;
    float *score = nullptr, *wdl = nullptr;
    int n_pos = 0;
    float norm = 0.f;
};

struct HostStage {
    int *stm = nullptr, *nstm = nullptr, *nnz = nullptr, *bucket = nullptr;
    float *score = nullptr, *wdl = nullptr;
};

enum Phase {
    PH_SORT = 0, PH_FT_FWD, PH_L1_FWD, PH_TAIL, PH_SMALL_WGRAD, PH_L1_WGRAD, PH_L1_DGRAD, PH_INV_INDEX, PH_FT_BWD,
    PH_ALLREDUCE, PH_OPT_FT, PH_OPT_SMALL, PH_COUNT
};
const char* const kPhaseNames[PH_COUNT] = {"bucket_sort", "ft_forward", "l1_forward", "tail", "small_wgrad", "l1_wgrad",
                                           "l1_dgrad_ftgrad", "inverse_index", "ft_backward", "allreduce", "opt_ft",
                                           "opt_small"};

}  // namespace

struct tb_trainer {
    tb_config cfg;
    std::string err;
    cudaStream_t stream = nullptr, copy_stream = nullptr;
    std::vector<Group> groups;
    float* grad_arena = nullptr;
    int64_t arena_len = 0, arena_reduce_len = 0;
    float* comb = nullptr;
    // reduced precision (bins/nnue_train/src/cli.rs:623-638): what each flag switches is in validate_config
    bool p_tf32 = false, p_ft16 = false, p_out16 = false, p_state16 = false;
    void* table_h = nullptr;          // fp16 forward table: folded table [N, F] (factorizer) or mirror of ft_w [N, F]
    void *pre_h[2] = {nullptr, nullptr}, *dft_h[2] = {nullptr, nullptr};  // fp16 pre-activations / loss-scaled dft rows
    void *ft_m_h = nullptr, *ft_v_h = nullptr;                           // fp16 moments of ft_w (scaled)
    unsigned long long* clamp_counter = nullptr;                         // device: dft elements clamped to +-65504 so far
    uint64_t clamp_elems = 0;                                            // dft elements written as fp16 so far
    float grad_unscale = 1.0f;        // 1 / (loss scale of the FT gradient rows of the last backward)
    int* tc_error = nullptr;          // device: raised by the tensor-core L1 kernel when a bounded wait ran out
    int* tc_error_pinned = nullptr;   // its host copy, refreshed with every loss read-back
    int Nt = 0, l1e = 0, l2in = 0, K = 0, max_tiles = 0, max_units = 0;
    uint64_t step_count = 0;
    // inputs
    DevBatch ring[2], slots[TB_NUM_SLOTS];
    HostStage stage[2];
    unsigned char* ring_psv[2] = {nullptr, nullptr};   // device: the 40-byte records of a batch fed as PackedSfenValue
    unsigned char* stage_psv[2] = {nullptr, nullptr};  // pinned staging for pageable record buffers
    cudaEvent_t ev_upload[2] = {nullptr, nullptr}, ev_consumed[2] = {nullptr, nullptr};
    bool upload_pending[2] = {false, false}, consumed_pending[2] = {false, false};
    uint64_t ring_step = 0;
    // workspace
    float *pre[2] = {nullptr, nullptr}, *dft[2] = {nullptr, nullptr}, *combined = nullptr;
    float *l1_out = nullptr, *dl1 = nullptr, *net_output = nullptr, *dy = nullptr;
    float *tail_a = nullptr, *tail_b = nullptr, *tail_c = nullptr;  // LS: l2_input, dl2_out, l2_acted; Simple: l1_acted, dl2_pre, l2_acted
    double *loss_partials = nullptr, *loss_acc = nullptr, *wrm_weight_sum = nullptr;
    int *order = nullptr, *n_tiles = nullptr, *seg_start = nullptr;
    TileDesc* tiles = nullptr;
    float *small_partials = nullptr, *l1w_partials = nullptr, *bias_partials = nullptr, *l1_weff = nullptr;
    int *feat_counts = nullptr, *feat_offsets = nullptr, *feat_cursor = nullptr, *feat_lists = nullptr;
    int *sort_hist = nullptr, *items = nullptr, *item_seg = nullptr, *bwd_plan = nullptr, *fwd_work = nullptr, *bwd_slice = nullptr;
    int dgrad_rows = 0;
    int n_sm = 148;
    cudaStream_t comm_stream = nullptr;  // data parallel: all-reduces behind the FT weight gradient
    cudaStream_t opt_stream = nullptr;   // data parallel: FT row updates behind their all-reduces
    cudaEvent_t ev_part[AR_PARTS_MAX] = {}, ev_reduced[AR_PARTS_MAX] = {}, ev_comm_done = nullptr, ev_opt_done = nullptr;
    bool ar_pipelined = false;
    bool opt_begun = false;        // this step's optimizer scalars are out (step_count already incremented)
    bool ft_rows_updated = false;  // this step's real FT rows were updated behind their all-reduces
    bool slice_fwd = false;  // this step's forward ran slice-resident (its row codes are in fwd_work)
    bool poisoned = false;   // a step failed after its optimizer had begun: parameters are part old, part new
    float* bwd_partial = nullptr;
    float* bwd_slabs = nullptr;  // partial gradient slabs of slices that several blocks share (ft_slice_bwd.cu)
    int last_n = 0;
    // loss ring (AsyncLossRing, trainer_common.rs:909-1000)
    double* loss_pinned[2] = {nullptr, nullptr};
    cudaEvent_t ev_loss[2] = {nullptr, nullptr};
    uint64_t loss_step = 0;
    bool loss_primed = false;
    // timing
    cudaEvent_t ev_t0 = nullptr, ev_t1 = nullptr;
    bool profile = false;
    cudaEvent_t ph_start[PH_COUNT], ph_stop[PH_COUNT];
    bool ph_used[PH_COUNT];
    double ph_ms[PH_COUNT];
    int64_t ph_launches[PH_COUNT];
    int64_t launches = 0;
    // data parallel
    void* comm = nullptr;
    PeerExchange* px = nullptr;  // TB_DP_PEER_COPY
    // TATARA_DP_TRACE: timing events of the data-parallel pipeline of one step (diagnostics)
    bool dp_trace = false;
    int dp_trace_parts = 0;
    cudaEvent_t tr_start = nullptr, tr_part[AR_PARTS_MAX] = {}, tr_red[AR_PARTS_MAX] = {}, tr_opt0[AR_PARTS_MAX] = {}, tr_opt1[AR_PARTS_MAX] = {}, tr_done = nullptr;
};

namespace {

int fail(tb_trainer* t, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (t) t->err = buf; else g_create_error = buf;
    return code;
}

#define CU(t, call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail(t, e_ == cudaErrorMemoryAllocation ? TB_ERR_OUT_OF_MEMORY : TB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); } while (0)

template <typename T>
cudaError_t dalloc(T** p, size_t n) {
    cudaError_t e = cudaMalloc((void**)p, (n ? n : 1) * sizeof(T));
    if (e == cudaSuccess) e = cudaMemset(*p, 0, (n ? n : 1) * sizeof(T));
    return e;
}

// start-up handshake of the peer exchange: `bytes` bytes per rank between host buffers, through NCCL
int nccl_host_allgather(void* ctx, const void* send, void* recv, size_t bytes) {
    tb_trainer* t = static_cast<tb_trainer*>(ctx);
    unsigned char *ds = nullptr, *dr = nullptr;
    int rc = -1;
    if (cudaMalloc((void**)&ds, bytes) == cudaSuccess && cudaMalloc((void**)&dr, bytes * t->cfg.world_size) == cudaSuccess &&
        cudaMemcpy(ds, send, bytes, cudaMemcpyHostToDevice) == cudaSuccess &&
        g_nccl.AllGather(ds, dr, bytes, /*ncclUint8*/ 1, t->comm, t->stream) == 0 && cudaStreamSynchronize(t->stream) == cudaSuccess &&
        cudaMemcpy(recv, dr, bytes * t->cfg.world_size, cudaMemcpyDeviceToHost) == cudaSuccess)
        rc = 0;
    cudaFree(ds); cudaFree(dr);
    return rc;
}

Group* find_group(tb_trainer* t, const char* name) {
    if (!name) return nullptr;
    for (auto& g : t->groups)
        if (g.name == name) return &g;
    return nullptr;
}

// radam_compute_step_size_denom (pointwise/radam_step.rs:63-86) and OptimizerKind::step_size_denom
// (crates/nnue-train/src/optimizer.rs:63-93)
void optimizer_scalars(int kind, uint64_t step, float* step_size, int* denom, float* beta1) {
    const float b1 = kind == TB_OPT_RANGER ? 0.99f : 0.9f;
    *beta1 = b1;
    if (kind == TB_OPT_ADAMW) { *step_size = 1.0f; *denom = 1; return; }
    const float step_f = (float)step;
    const float beta2_t = powf(BETA2, step_f);
    const float n_sma_max = 2.0f / (1.0f - BETA2) - 1.0f;
    const float n_sma = n_sma_max - 2.0f * step_f * beta2_t / (1.0f - beta2_t);
    const float bc1 = 1.0f - powf(b1, step_f);
    if (n_sma > N_SMA_THRESHOLD) {
        const float p1 = (n_sma - 4.0f) / (n_sma_max - 4.0f);
        const float p2 = (n_sma - 2.0f) / n_sma;
        const float p3 = n_sma_max / (n_sma_max - 2.0f);
        *step_size = sqrtf((1.0f - beta2_t) * p1 * p2 * p3) / bc1;
    } else {
        *step_size = 1.0f / bc1;
    }
    *denom = n_sma > N_SMA_THRESHOLD ? 1 : 0;
}

struct PhaseScope {
    tb_trainer* t;
    int ph;
    PhaseScope(tb_trainer* t_, int ph_) : t(t_), ph(ph_) {
        if (t->profile) { cudaEventRecord(t->ph_start[ph], t->stream); }
    }
    void done(int launches) {
        t->launches += launches;
        if (t->profile) {
            cudaEventRecord(t->ph_stop[ph], t->stream);
            t->ph_used[ph] = true;
            t->ph_launches[ph] += launches;
        }
    }
};

void profile_collect(tb_trainer* t) {
    if (!t->profile) return;
    cudaStreamSynchronize(t->stream);
    for (int i = 0; i < PH_COUNT; ++i)
        if (t->ph_used[i]) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, t->ph_start[i], t->ph_stop[i]) == cudaSuccess) t->ph_ms[i] += ms;
            t->ph_used[i] = false;
        }
}

int check_batch(tb_trainer* t, const tb_batch* b) {
    if (!b) return fail(t, TB_ERR_INVALID_ARGUMENT, "batch is NULL");
    if (b->n_pos < 0) return fail(t, TB_ERR_INVALID_ARGUMENT, "batch.n_pos is negative (%d)", b->n_pos);
    if (b->n_pos == 0) return TB_OK;
    // trainer_layerstack.rs:79-89
    if (b->n_pos % 16 != 0)
        return fail(t, TB_ERR_INVALID_ARGUMENT, "batch.n_pos must be a multiple of 16 (got %d)", b->n_pos);
    // trainer_layerstack.rs:608-621
    if (b->n_pos > t->cfg.batch_capacity)
        return fail(t, TB_ERR_INVALID_ARGUMENT,
                    "batch %d exceeds workspace capacity %d (the workspace is allocated once at creation)", b->n_pos,
                    t->cfg.batch_capacity);
    if (!b->stm_indices || !b->nstm_indices || !b->nnz || !b->score || !b->wdl)
        return fail(t, TB_ERR_INVALID_ARGUMENT, "batch has a NULL input array");
    if (t->cfg.arch == TB_ARCH_LAYERSTACK && !b->bucket_idx)
        return fail(t, TB_ERR_INVALID_ARGUMENT, "LayerStack needs batch.bucket_idx");
    return TB_OK;
}

bool is_pinned(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeHost;
}

// Copies one host batch into a device batch on `cs`.  Pinned caller memory is copied directly; pageable
// memory goes through the library's pinned staging buffers first.
int upload_batch(tb_trainer* t, const tb_batch* b, DevBatch* d, HostStage* st, cudaStream_t cs) {
    const size_t n = (size_t)b->n_pos, A = (size_t)t->cfg.max_active;
    const bool ls = t->cfg.arch == TB_ARCH_LAYERSTACK;
    struct Item { void* dst; const void* src; void* stage; size_t bytes; } items[6] = {
        {d->stm, b->stm_indices, st ? st->stm : nullptr, n * A * 4}, {d->nstm, b->nstm_indices, st ? st->nstm : nullptr, n * A * 4},
        {d->nnz, b->nnz, st ? st->nnz : nullptr, n * 4},             {d->bucket, b->bucket_idx, st ? st->bucket : nullptr, n * 4},
        {d->score, b->score, st ? st->score : nullptr, n * 4},       {d->wdl, b->wdl, st ? st->wdl : nullptr, n * 4}};
    for (int i = 0; i < 6; ++i) {
        if (i == 3 && !ls) continue;
        const void* src = items[i].src;
        if (items[i].stage && !is_pinned(src)) {
            memcpy(items[i].stage, src, items[i].bytes);
            src = items[i].stage;
        }
        CU(t, cudaMemcpyAsync(items[i].dst, src, items[i].bytes, cudaMemcpyHostToDevice, cs));
    }
    d->n_pos = b->n_pos;
    d->norm = b->per_pos_norm != 0.f ? b->per_pos_norm : 1.0f / ((float)b->n_pos * (float)t->cfg.world_size);
    return TB_OK;
}

LossParams make_loss(const tb_loss* l, float lambda, float norm) {
    LossParams p;
    p.kind = l->kind;
    p.scale = l->scale;
    p.nnue2score = l->nnue2score;
    p.in_scaling = l->in_scaling;
    p.in_offset = l->in_offset;
    p.target_offset = l->target_offset;
    p.target_scaling = l->target_scaling;
    p.lambda = lambda;
    p.norm = norm;
    // LossKind::wrm_extended (crates/nnue-train/src/trainer.rs:127-137)
    p.extended = l->kind == TB_LOSS_WRM && !(l->pow_exp == 2.0f && l->qp_asymmetry == 0.0f && l->weight_boost_w1 == 0.0f);
    p.pow_exp = l->pow_exp;
    p.qp_asymmetry = l->qp_asymmetry;
    p.w1 = l->weight_boost_w1;
    p.w2 = l->weight_boost_w2;
    return p;
}

int check_loss(tb_trainer* t, const tb_loss* l) {
    if (!l) return fail(t, TB_ERR_INVALID_ARGUMENT, "loss is NULL");
    if (l->kind == TB_LOSS_SIGMOID) {
        if (!(l->scale > 0.f) || !isfinite(l->scale))
            return fail(t, TB_ERR_INVALID_ARGUMENT, "loss scale must be finite and > 0 (got %g)", l->scale);
        return TB_OK;
    }
    if (l->kind != TB_LOSS_WRM) return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown loss kind %d", l->kind);
    if (!(l->nnue2score > 0.f) || !(l->in_scaling > 0.f) || !(l->target_scaling > 0.f))
        return fail(t, TB_ERR_INVALID_ARGUMENT, "wrm nnue2score / in_scaling / target_scaling must be > 0");
    // LossKind::wrm_extended (crates/nnue-train/src/trainer.rs:127-137): its per-position weights are normalised by their sum
    // over the batch, which with several ranks would have to be the sum over all ranks' shards
    if ((l->pow_exp != 2.0f || l->qp_asymmetry != 0.0f || l->weight_boost_w1 != 0.0f) && t->cfg.world_size > 1)
        return fail(t, TB_ERR_UNSUPPORTED, "the extended WRM loss (pow_exp / qp_asymmetry / weight boost) is built for one GPU only");
    if (!(l->pow_exp > 0.0f) || !isfinite(l->pow_exp)) return fail(t, TB_ERR_INVALID_ARGUMENT, "wrm pow_exp must be finite and > 0");
    return TB_OK;
}

// ---- the step ------------------------------------------------------------------------------------------
int run_forward(tb_trainer* t, const DevBatch& d, const tb_loss* loss, float lambda, int backward) {
    const tb_config& c = t->cfg;
    const int B = d.n_pos, F = c.ft_out, N = c.ft_in, A = c.max_active;
    const bool ls = c.arch == TB_ARCH_LAYERSTACK;
    const void* table = t->p_ft16 ? t->table_h : (c.ft_factorize ? (const void*)t->comb : (const void*)t->groups[0].w);
    void* pre0 = t->p_out16 ? t->pre_h[0] : (void*)t->pre[0];
    void* pre1 = t->p_out16 ? t->pre_h[1] : (void*)t->pre[1];
    t->last_n = B;
    if (backward) { t->opt_begun = false; t->ft_rows_updated = false; }
    { PhaseScope p(t, PH_SORT);
      // positions by bucket (order, tiles, units) and items of both perspectives by the king-bucket slice of the FT table
      int n = launch_step_sorts(t->stream, ls ? d.bucket : nullptr, B, ls ? c.num_buckets : 0, t->order, t->tiles, t->n_tiles,
                                t->seg_start, t->max_tiles, d.stm, d.nstm, d.nnz, A, N, c.piece_inputs > 0 ? c.piece_inputs : N, 2,
                                t->items, t->item_seg, t->sort_hist);
      p.done(n); }
    { PhaseScope p(t, PH_FT_FWD);
      const int mode = (ls || c.activation == TB_ACT_PAIRWISE) ? 1 : (c.activation == TB_ACT_CRELU ? 2 : 3);
      const int rps = c.piece_inputs > 0 ? c.piece_inputs : N;
      t->slice_fwd = ft_forward_slice_supported(F, N, A, rps);
      if (t->slice_fwd)
          p.done(launch_ft_forward_slice(t->stream, mode, table, d.stm, d.nstm, d.nnz, t->groups[1].w, pre0, pre1,
                                         t->combined, t->items, t->item_seg, t->fwd_work, B, F, N, A, rps, FT_POST_SCALE, 2,
                                         t->p_ft16, t->p_out16));
      else
          p.done(launch_ft_forward(t->stream, mode, table, d.stm, d.nstm, d.nnz, t->groups[1].w, pre0, pre1, t->combined,
                                   t->items, B, F, N, A, FT_POST_SCALE, 2, t->p_ft16, t->p_out16)); }
    LossParams lp = make_loss(loss, lambda, d.norm);
    if (lp.extended) {  // the weight sum of this batch first (trainer_simple.rs:1430-1478 launches wrm_weight_sum before loss_wrm)
        PhaseScope p(t, PH_TAIL);
        lp.n_pos = (float)B;
        lp.weight_sum = t->wrm_weight_sum;
        p.done(launch_wrm_weight_sum(t->stream, d.score, B, lp, t->loss_partials, t->wrm_weight_sum));
    }
    if (ls) {
        { PhaseScope p(t, PH_L1_FWD);
          p.done(launch_l1_forward(t->stream, t->combined, F, t->order, t->tiles, t->n_tiles, t->max_tiles, t->groups[2].w,
                                   t->groups[3].w, t->groups[4].w, t->groups[5].w, t->l1_out, c.l1_out, c.num_buckets, t->l1_weff,
                                   t->p_tf32, t->tc_error)); }
        { PhaseScope p(t, PH_TAIL);
          p.done(launch_tail_layerstack(t->stream, t->l1_out, d.bucket, d.score, d.wdl, t->groups[6].w, t->groups[7].w,
                                        t->groups[8].w, t->groups[9].w, lp, B, c.l1_out, c.l2_out, c.num_buckets,
                                        t->net_output, t->dy, t->dl1, t->tail_a, t->tail_b, t->tail_c, t->loss_partials,
                                        t->loss_acc, backward)); }
    } else {
        { PhaseScope p(t, PH_L1_FWD);
          p.done(launch_l1_forward(t->stream, t->combined, t->K, t->order, t->tiles, t->n_tiles, t->max_tiles, nullptr, nullptr,
                                   t->groups[2].w, t->groups[3].w, t->l1_out, c.l1_out, 0, t->l1_weff)); }
        { PhaseScope p(t, PH_TAIL);
          p.done(launch_tail_simple(t->stream, t->l1_out, d.score, d.wdl, t->groups[4].w, t->groups[5].w, t->groups[6].w,
                                    t->groups[7].w, lp, c.activation == TB_ACT_SCRELU ? 1 : 0, B, c.l1_out, c.l2_out, t->net_output, t->dy, t->dl1,
                                    t->tail_a, t->tail_b, t->tail_c, t->loss_partials, t->loss_acc, backward)); }
    }
    return TB_OK;
}

static OptScalars ft_scalars(tb_trainer* t, float lr);

// lr >= 0: a full training step (the data-parallel pipeline may then update FT rows behind their all-reduces);
// lr < 0: gradients only
int run_backward(tb_trainer* t, const DevBatch& d, float lr) {
    const tb_config& c = t->cfg;
    const int B = d.n_pos, F = c.ft_out, N = c.ft_in, A = c.max_active;
    const bool ls = c.arch == TB_ARCH_LAYERSTACK;
    if (ls) {
        { PhaseScope p(t, PH_SMALL_WGRAD);
          p.done(launch_small_wgrad_layerstack(t->stream, t->order, t->seg_start, B, c.l1_out, c.l2_out, c.num_buckets, t->tail_a,
                                               t->tail_b, t->tail_c, t->dy, t->dl1, t->small_partials, t->groups[6].grad,
                                               t->groups[7].grad, t->groups[8].grad, t->groups[9].grad, t->groups[3].grad,
                                               t->groups[5].grad)); }
        { PhaseScope p(t, PH_L1_WGRAD);
          p.done(launch_l1_wgrad(t->stream, t->combined, F, t->dl1, t->order, t->tiles, t->n_tiles, t->max_tiles, c.l1_out,
                                 c.num_buckets, t->l1w_partials, t->groups[2].grad, t->groups[4].grad)); }
        { PhaseScope p(t, PH_L1_DGRAD);
          // fp16 dft rows carry gradient * 2^14 * batch (trainer_layerstack.rs:3617-3621); the FT weight gradient is summed
          // in that scale and the optimizer takes it out again
          const float dft_scale = t->p_out16 ? FT_DFT_FP16_BASE_SCALE * (float)B : 1.0f;
          t->grad_unscale = 1.0f / dft_scale;
          if (t->p_out16) t->clamp_elems += 2ull * (uint64_t)B * (uint64_t)F;
          p.done(launch_l1_dgrad_ftgrad(t->stream, 1, t->dl1, t->order, t->tiles, t->n_tiles, t->max_tiles, t->groups[2].w,
                                        t->groups[4].w, t->p_out16 ? t->pre_h[0] : (void*)t->pre[0],
                                        t->p_out16 ? t->pre_h[1] : (void*)t->pre[1], t->groups[1].w, FT_POST_SCALE, B, F, c.l1_out,
                                        c.num_buckets, t->p_out16 ? t->dft_h[0] : (void*)t->dft[0],
                                        t->p_out16 ? t->dft_h[1] : (void*)t->dft[1], t->bias_partials, t->groups[1].grad,
                                        t->dgrad_rows, t->p_out16, dft_scale, t->clamp_counter)); }
    } else {
        { PhaseScope p(t, PH_SMALL_WGRAD);
          p.done(launch_small_wgrad_simple(t->stream, t->order, t->seg_start, B, c.l1_out, c.l2_out, t->tail_a, t->tail_b,
                                           t->tail_c, t->dy, t->dl1, t->small_partials, t->groups[4].grad, t->groups[5].grad,
                                           t->groups[6].grad, t->groups[7].grad, t->groups[3].grad)); }
        { PhaseScope p(t, PH_L1_WGRAD);
          p.done(launch_l1_wgrad(t->stream, t->combined, t->K, t->dl1, t->order, t->tiles, t->n_tiles, t->max_tiles, c.l1_out, 0,
                                 t->l1w_partials, nullptr, t->groups[2].grad)); }
        { PhaseScope p(t, PH_L1_DGRAD);
          p.done(launch_l1_dgrad_ftgrad(t->stream, c.activation == TB_ACT_PAIRWISE ? 1 : (c.activation == TB_ACT_CRELU ? 2 : 3), t->dl1, t->order, t->tiles, t->n_tiles,
                                        t->max_tiles, nullptr, t->groups[2].w, t->pre[0], t->pre[1], t->groups[1].w,
                                        FT_POST_SCALE, B, F, c.l1_out, 0, t->dft[0], t->dft[1], t->bias_partials,
                                        t->groups[1].grad, t->dgrad_rows)); }
    }
    // slice-resident path when this step's forward was; the generic kernels then run only for a batch with a row outside
    // its item's slice (device-side gate)
    const int rps = c.piece_inputs > 0 ? c.piece_inputs : N;
    const void* dft0 = t->p_out16 ? t->dft_h[0] : (const void*)t->dft[0];
    const void* dft1 = t->p_out16 ? t->dft_h[1] : (const void*)t->dft[1];
    const bool slice_bwd = t->slice_fwd && t->bwd_slice != nullptr;
    const int* gate = slice_bwd ? ft_slice_outside_flag(t->fwd_work, 2 * B, N, rps) : nullptr;
    { PhaseScope p(t, PH_INV_INDEX);
      int n = 0;
      if (slice_bwd) n += launch_inverse_slice(t->stream, t->item_seg, t->fwd_work, t->bwd_slice, B, A, N, rps, 2);
      n += launch_inverse_index(t->stream, gate, d.stm, d.nstm, d.nnz, B, A, N, 2, t->feat_counts, t->feat_offsets, t->feat_cursor,
                                t->feat_lists);
      p.done(n); }
    { PhaseScope p(t, PH_FT_BWD);
      int n = launch_ft_backward_split(t->stream, gate, dft0, dft1, t->feat_offsets, t->feat_lists, B, A, N, F, 2,
                                       t->bwd_plan, t->bwd_partial, t->groups[0].grad, t->p_out16);
      if (slice_bwd) {
          // Data parallel: the slices are done in several launches (ar_parts_for) and the gradient rows of each part are all-reduced on a
          // second stream while the next part is computed (the small groups, ready since the dense backward, ride with the
          // first part, the loss with the last).  Whichever path wrote the rows (the gated generic kernels come first), they
          // are final when the part's event is recorded.
          const int n_slices = (N + rps - 1) / rps;
          const int strips = t->p_out16 ? F / 64 : F / 32;
          const int parts = c.world_size > 1 ? ar_parts_for(n_slices, strips, t->n_sm) : 1;
          const bool pipeline = parts > 1;
          const int64_t ft_off = t->groups[0].grad - t->grad_arena;
          int rc = 0;
          const bool trace = t->dp_trace && pipeline && t->step_count == 20;
          if (trace) { t->dp_trace_parts = parts; CU(t, cudaEventRecord(t->tr_start, t->stream)); }
          for (int part = 0; part < parts; ++part) {
              // equal parts: shorter last parts (tapered sizes, or whole waves with a one-wave last part) were measured slower
              // on two and four GPUs, with NCCL and with the peer exchange
              const int k0 = (int)((int64_t)n_slices * part / parts), k1 = (int)((int64_t)n_slices * (part + 1) / parts);
              n += launch_ft_backward_slice(t->stream, dft0, dft1, t->fwd_work, t->bwd_slice, B, A, N, F, rps, 2, k0, k1 - k0,
                                            t->groups[0].grad, t->bwd_slabs, t->p_out16);
              if (!pipeline) continue;
              CU(t, cudaEventRecord(t->ev_part[part], t->stream));
              if (trace) CU(t, cudaEventRecord(t->tr_part[part], t->stream));
              CU(t, cudaStreamWaitEvent(t->comm_stream, t->ev_part[part], 0));
              const int64_t e0 = part == 0 ? 0 : ft_off + (int64_t)(k0 * rps < N ? k0 * rps : N) * F;
              const int64_t e1 = ft_off + (int64_t)(k1 * rps < N ? k1 * rps : N) * F;
              if (t->px) {
                  // copy engines and peer mappings: the reduce kernel on the communication stream, the consumer's waits on
                  // the optimizer stream
                  if (part == 0) px_begin_step(t->px);
                  std::string e;
                  if (px_exchange_part(t->px, part, e0, e1, part == parts - 1, t->ev_part[part], t->comm_stream, t->opt_stream, &n, &e) != 0)
                      return fail(t, TB_ERR_CUDA, "%s", e.c_str());
              } else {
                  if (rc == 0) rc = g_nccl.GroupStart();
                  if (rc == 0) rc = g_nccl.AllReduce(t->grad_arena + e0, t->grad_arena + e0, (size_t)(e1 - e0), /*ncclFloat*/ 7, /*ncclSum*/ 0, t->comm, t->comm_stream);
                  if (rc == 0 && part == parts - 1) rc = g_nccl.AllReduce(t->loss_acc, t->loss_acc, 1, /*ncclDouble*/ 8, 0, t->comm, t->comm_stream);
                  const int rc2 = g_nccl.GroupEnd();
                  if (rc == 0) rc = rc2;
              }
              if (trace) { CU(t, cudaEventRecord(t->tr_red[part], t->comm_stream)); CU(t, cudaEventRecord(t->tr_opt0[part], t->opt_stream)); }
              if (rc == 0 && lr >= 0.0f) {
                  // consumer side of the pipeline: the optimizer of this part's real rows follows its all-reduce on the
                  // same stream, next to the gradient launch of the next part (and alone on the GPU behind the last)
                  // (a third stream: the next part's all-reduce does not wait for this part's optimizer)
                  const OptScalars sc = ft_scalars(t, lr);
                  Group& g = t->groups[0];
                  const int r0 = k0 * rps, r1 = k1 * rps < N ? k1 * rps : N;
                  CU(t, cudaEventRecord(t->ev_reduced[part], t->comm_stream));
                  CU(t, cudaStreamWaitEvent(t->opt_stream, t->ev_reduced[part], 0));
                  const size_t msz = t->p_state16 ? 2 : 4, e0r = (size_t)r0 * F;
                  void* gm = t->p_state16 ? t->ft_m_h : (void*)g.m;
                  void* gv = t->p_state16 ? t->ft_v_h : (void*)g.v;
                  if (c.ft_factorize)
                      n += launch_radam_factorized_rows(t->opt_stream, g.w, gm, gv, g.grad, g.slow, N, c.piece_inputs, F, k0, k1, sc,
                                                        t->p_state16);
                  else
                      n += launch_radam(t->opt_stream, g.w + e0r, (char*)gm + e0r * msz, (char*)gv + e0r * msz, g.grad + e0r,
                                        c.optimizer == TB_OPT_RANGER ? g.slow + e0r : g.slow, (int64_t)(r1 - r0) * F, sc, t->p_state16,
                                        t->p_ft16 ? (char*)t->table_h + e0r * 2 : nullptr);
                  t->ft_rows_updated = true;
                  if (trace) CU(t, cudaEventRecord(t->tr_opt1[part], t->opt_stream));
              }
          }
          if (pipeline) {
              if (rc != 0) return fail(t, TB_ERR_NCCL, "ncclAllReduce: %s", g_nccl.GetErrorString(rc));
              if (t->ft_rows_updated || t->px) {  // the optimizer stream (with the peer exchange: its waits) joins the communication stream
                  CU(t, cudaEventRecord(t->ev_opt_done, t->opt_stream));
                  CU(t, cudaStreamWaitEvent(t->comm_stream, t->ev_opt_done, 0));
              }
              if (t->px) {
                  std::string e;
                  if (px_join(t->px, t->comm_stream, &e) != 0) return fail(t, TB_ERR_CUDA, "%s", e.c_str());
              }
              CU(t, cudaEventRecord(t->ev_comm_done, t->comm_stream));
              if (trace) {
                  CU(t, cudaEventRecord(t->tr_done, t->comm_stream));
                  CU(t, cudaEventSynchronize(t->tr_done));
                  fprintf(stderr, "[dp trace rank %d] ms after the first gradient launch:", c.rank);
                  for (int q = 0; q < parts; ++q) {
                      float a = 0, b = 0, d0 = 0, d1 = 0;
                      cudaEventElapsedTime(&a, t->tr_start, t->tr_part[q]); cudaEventElapsedTime(&b, t->tr_start, t->tr_red[q]);
                      cudaEventElapsedTime(&d0, t->tr_start, t->tr_opt0[q]); cudaEventElapsedTime(&d1, t->tr_start, t->tr_opt1[q]);
                      fprintf(stderr, "  part %d: gradient %.3f reduced %.3f published %.3f rows updated %.3f;", q, a, b, d0, d1);
                  }
                  float e2 = 0;
                  cudaEventElapsedTime(&e2, t->tr_start, t->tr_done);
                  fprintf(stderr, "  all done %.3f\n", e2);
              }
              t->ar_pipelined = true;
          }
      }
      p.done(n); }
    return TB_OK;
}

// sum of the gradient arena (and of the loss) over the data-parallel ranks
int run_allreduce(tb_trainer* t) {
    if (t->cfg.world_size <= 1) return TB_OK;
    PhaseScope p(t, PH_ALLREDUCE);
    if (t->ar_pipelined) {  // issued part by part behind the FT weight gradient: only the tail is waited for here
        t->ar_pipelined = false;
        CU(t, cudaStreamWaitEvent(t->stream, t->ev_comm_done, 0));
        p.done(1);  // counted so that the wait shows up in the per-phase report
        return TB_OK;
    }
    int rc = g_nccl.GroupStart();
    if (rc == 0) rc = g_nccl.AllReduce(t->grad_arena, t->grad_arena, (size_t)t->arena_reduce_len, /*ncclFloat*/ 7, /*ncclSum*/ 0, t->comm, t->stream);
    if (rc == 0) rc = g_nccl.AllReduce(t->loss_acc, t->loss_acc, 1, /*ncclDouble*/ 8, 0, t->comm, t->stream);
    const int rc2 = g_nccl.GroupEnd();
    if (rc == 0) rc = rc2;
    p.done(2);
    if (rc != 0) return fail(t, TB_ERR_NCCL, "ncclAllReduce: %s", g_nccl.GetErrorString(rc));
    return TB_OK;
}

// The step's optimizer scalars; the first call of a step increments step_count (before the scalars are computed,
// trainer_layerstack.rs:4078-4081), run_optimizer ends the step.
static OptScalars optimizer_step_scalars(tb_trainer* t) {
    const tb_config& c = t->cfg;
    if (!t->opt_begun) {
        t->step_count += 1;
        t->opt_begun = true;
    }
    OptScalars sc;
    optimizer_scalars(c.optimizer, t->step_count, &sc.step_size, &sc.denom, &sc.beta1);
    sc.beta2 = BETA2;
    sc.eps = EPS;
    sc.alpha = RANGER_ALPHA;
    sc.lerp = (c.optimizer == TB_OPT_RANGER && t->step_count % RANGER_K == 0) ? 1 : 0;
    return sc;
}

static OptScalars ft_scalars(tb_trainer* t, float lr) {
    OptScalars sc = optimizer_step_scalars(t);
    const Group& g = t->groups[0];
    sc.lr = lr * t->cfg.lr_mult_ft;
    sc.decay = t->cfg.wd_ft;
    sc.min_w = -g.clamp;
    sc.max_w = g.clamp;
    sc.grad_scale = t->p_out16 ? t->grad_unscale : 1.0f;
    return sc;
}

int run_optimizer(tb_trainer* t, float lr) {
    const tb_config& c = t->cfg;
    const bool ls = c.arch == TB_ARCH_LAYERSTACK;
    OptScalars sc = optimizer_step_scalars(t);
    t->opt_begun = false;
    const float wd[3] = {c.wd_ft, ls ? c.wd_dense : c.wd_ft, ls ? c.wd_bias : c.wd_ft};
    const float lm[3] = {c.lr_mult_ft, ls ? c.lr_mult_dense : c.lr_mult_ft, ls ? c.lr_mult_bias : c.lr_mult_ft};
    {
        PhaseScope p(t, PH_OPT_FT);
        Group& g = t->groups[0];
        sc.lr = lr * lm[0];
        sc.decay = wd[0];
        sc.min_w = -g.clamp;
        sc.max_w = g.clamp;
        sc.grad_scale = t->p_out16 ? t->grad_unscale : 1.0f;
        void* gm = t->p_state16 ? t->ft_m_h : (void*)g.m;
        void* gv = t->p_state16 ? t->ft_v_h : (void*)g.v;
        void* fwd_table = t->p_ft16 ? t->table_h : (void*)t->comb;  // what the forward reads: written in the same pass
        if (t->ft_rows_updated) {
            // data parallel: the real rows were updated part by part behind their all-reduces; what is left are the
            // virtual rows and the folded table
            t->ft_rows_updated = false;
            if (c.ft_factorize)
                p.done(launch_radam_factorized_fold(t->stream, g.w, gm, gv, g.grad, g.slow, fwd_table, c.ft_in, c.piece_inputs, c.ft_out, sc,
                                                    t->p_state16, t->p_ft16));
            else
                p.done(0);
        } else if (c.ft_factorize)
            p.done(launch_radam_factorized(t->stream, g.w, gm, gv, g.grad, g.slow, fwd_table, c.ft_in, c.piece_inputs, c.ft_out, sc,
                                           t->p_state16, t->p_ft16));
        else
            p.done(launch_radam(t->stream, g.w, gm, gv, g.grad, g.slow, g.len, sc, t->p_state16, t->p_ft16 ? t->table_h : nullptr));
        sc.grad_scale = 1.0f;  // the small groups' gradients are never scaled
    }
    {
        PhaseScope p(t, PH_OPT_SMALL);
        SmallGroups sg;
        sg.n = 0;
        int max_n = 0;
        for (size_t i = 1; i < t->groups.size(); ++i) {
            Group& g = t->groups[i];
            SmallGroup& s = sg.g[sg.n++];
            s.w = g.w; s.m = g.m; s.v = g.v; s.slow = g.slow; s.grad = g.grad;
            s.n = (int)g.len;
            s.lr = lr * lm[g.kind];
            s.decay = wd[g.kind];
            s.min_w = -g.clamp;
            s.max_w = g.clamp;
            if (s.n > max_n) max_n = s.n;
        }
        p.done(launch_radam_small(t->stream, sg, max_n, sc));
    }
    return TB_OK;
}

// Waits for a loss read-back.  With the peer exchange a lost peer shows as a stream that never finishes (its flags never
// arrive): the wait then has a deadline, after which the handle refuses further steps.
int wait_loss_event(tb_trainer* t, cudaEvent_t ev) {
    if (!t->px) { CU(t, cudaEventSynchronize(ev)); return TB_OK; }
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t e = cudaEventQuery(ev);
        if (e == cudaSuccess) return TB_OK;
        if (e != cudaErrorNotReady) return fail(t, TB_ERR_CUDA, "cudaEventQuery: %s", cudaGetErrorString(e));
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(PEER_DEADLINE_S)) {
            t->poisoned = true;
            return fail(t, TB_ERR_TIMEOUT, "a data-parallel step did not finish within %d s: a peer rank is gone or stuck", PEER_DEADLINE_S);
        }
        std::this_thread::yield();
    }
}

// queues the read-back of this step's loss and returns the previous one (AsyncLossRing::read_and_queue_next)
int loss_ring_next(tb_trainer* t, double* out) {
    const int cur = (int)(t->loss_step % 2);
    if (t->tc_error) {
        if (*t->tc_error_pinned) return fail(t, TB_ERR_CUDA, "the tensor-core L1 kernel gave up waiting for its MMAs (an earlier step's results are invalid)");
        CU(t, cudaMemcpyAsync(t->tc_error_pinned, t->tc_error, sizeof(int), cudaMemcpyDeviceToHost, t->stream));
    }
    CU(t, cudaMemcpyAsync(t->loss_pinned[cur], t->loss_acc, sizeof(double), cudaMemcpyDeviceToHost, t->stream));
    CU(t, cudaEventRecord(t->ev_loss[cur], t->stream));
    double returned = 0.0;
    if (t->loss_primed) {
        const int prev = (int)((t->loss_step + 1) % 2);
        { const int wrc = wait_loss_event(t, t->ev_loss[prev]); if (wrc != TB_OK) return wrc; }
        returned = *t->loss_pinned[prev];
    } else {
        t->loss_primed = true;
    }
    t->loss_step += 1;
    if (out) *out = returned;
    return TB_OK;
}

int step_on(tb_trainer* t, const DevBatch& d, float lr, float lambda, const tb_loss* loss, double* loss_prev) {
    if (t->poisoned)
        return fail(t, TB_ERR_CUDA, "an earlier step failed after its optimizer had begun; the parameters are inconsistent: "
                                    "destroy the handle and restore a checkpoint");
    int rc = run_forward(t, d, loss, lambda, 1);
    if (rc == TB_OK) rc = run_backward(t, d, lr);
    if (rc == TB_OK) rc = run_allreduce(t);
    // Up to here a failed step leaves the parameters and step_count untouched, unless the data-parallel pipeline had
    // already sent the optimizer behind the first gradient parts (opt_begun): then some FT rows carry this step's update
    // and a retry would apply it twice, so the handle refuses further steps.
    if (rc != TB_OK && t->opt_begun) t->poisoned = true;
    if (rc == TB_OK) {
        rc = run_optimizer(t, lr);
        if (rc == TB_OK && cudaGetLastError() != cudaSuccess) rc = fail(t, TB_ERR_CUDA, "a kernel launch of the step failed");
        if (rc != TB_OK) t->poisoned = true;
    }
    if (rc != TB_OK) return rc;
    rc = loss_ring_next(t, loss_prev);
    profile_collect(t);
    return rc;
}

// uploads into ring slot `s` on the copy stream and makes the compute stream wait for it
int ring_upload(tb_trainer* t, const tb_batch* b, int* slot_out) {
    const int s = (int)(t->ring_step % 2);
    // the previous upload from this staging slot must have left the host buffers
    if (t->upload_pending[s]) { CU(t, cudaEventSynchronize(t->ev_upload[s])); t->upload_pending[s] = false; }
    // the compute that read this device slot two steps ago must be done before it is overwritten
    if (t->consumed_pending[s]) { CU(t, cudaStreamWaitEvent(t->copy_stream, t->ev_consumed[s], 0)); }
    int rc = upload_batch(t, b, &t->ring[s], &t->stage[s], t->copy_stream);
    if (rc != TB_OK) return rc;
    CU(t, cudaEventRecord(t->ev_upload[s], t->copy_stream));
    t->upload_pending[s] = true;
    CU(t, cudaStreamWaitEvent(t->stream, t->ev_upload[s], 0));
    // a caller-owned pinned buffer of the OTHER slot may be reused by the caller once this call returns
    const int o = s ^ 1;
    if (t->upload_pending[o]) { CU(t, cudaEventSynchronize(t->ev_upload[o])); t->upload_pending[o] = false; }
    t->ring_step += 1;
    *slot_out = s;
    return TB_OK;
}

// The same for a batch given as PackedSfenValue records: 40 bytes per position cross the bus, the indices, buckets and
// targets are produced on the device by k_psv_extract, on the copy stream, so that decode and extraction of batch k + 1
// overlap the compute of batch k (the work of the reference's dataloader workers,
// crates/nnue-train/src/dataloader.rs:1303-1407).
int ring_upload_psv(tb_trainer* t, int feature_set, const uint8_t* psv, int n_pos, int* slot_out) {
    const int s = (int)(t->ring_step % 2);
    if (t->upload_pending[s]) { CU(t, cudaEventSynchronize(t->ev_upload[s])); t->upload_pending[s] = false; }
    if (t->consumed_pending[s]) { CU(t, cudaStreamWaitEvent(t->copy_stream, t->ev_consumed[s], 0)); }
    const void* src = psv;
    const size_t bytes = (size_t)n_pos * 40;
    if (!is_pinned(psv)) { memcpy(t->stage_psv[s], psv, bytes); src = t->stage_psv[s]; }
    CU(t, cudaMemcpyAsync(t->ring_psv[s], src, bytes, cudaMemcpyHostToDevice, t->copy_stream));
    DevBatch& d = t->ring[s];
    const int n = launch_psv_extract(t->copy_stream, feature_set, t->ring_psv[s], n_pos, d.stm, d.nstm, d.nnz,
                                     t->cfg.arch == TB_ARCH_LAYERSTACK ? d.bucket : nullptr, d.score, d.wdl);
    if (n < 0) return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown feature set id %d", feature_set);
    t->launches += n;
    d.n_pos = n_pos;
    d.norm = 1.0f / ((float)n_pos * (float)t->cfg.world_size);
    CU(t, cudaEventRecord(t->ev_upload[s], t->copy_stream));
    t->upload_pending[s] = true;
    CU(t, cudaStreamWaitEvent(t->stream, t->ev_upload[s], 0));
    const int o = s ^ 1;
    if (t->upload_pending[o]) { CU(t, cudaEventSynchronize(t->ev_upload[o])); t->upload_pending[o] = false; }
    t->ring_step += 1;
    *slot_out = s;
    return TB_OK;
}

void free_all(tb_trainer* t) {
    if (!t) return;
    if (t->stream) cudaStreamSynchronize(t->stream);
    if (t->copy_stream) cudaStreamSynchronize(t->copy_stream);
    if (t->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(t->comm);
    for (auto& g : t->groups) { cudaFree(g.w); cudaFree(g.m); cudaFree(g.v); cudaFree(g.slow); }
    px_destroy(t->px);
    cudaFree(t->grad_arena);
    cudaFree(t->comb);
    cudaFree(t->table_h); cudaFree(t->ft_m_h); cudaFree(t->ft_v_h); cudaFree(t->clamp_counter);
    cudaFree(t->tc_error); cudaFreeHost(t->tc_error_pinned);
    for (int i = 0; i < 2; ++i) { cudaFree(t->pre_h[i]); cudaFree(t->dft_h[i]); }
    auto free_batch = [](DevBatch& d) { cudaFree(d.stm); cudaFree(d.nstm); cudaFree(d.nnz); cudaFree(d.bucket); cudaFree(d.score); cudaFree(d.wdl); };
    for (auto& d : t->ring) free_batch(d);
    for (auto& d : t->slots) free_batch(d);
    for (int i = 0; i < 2; ++i) { cudaFree(t->ring_psv[i]); cudaFreeHost(t->stage_psv[i]); }
    for (auto& s : t->stage) { cudaFreeHost(s.stm); cudaFreeHost(s.nstm); cudaFreeHost(s.nnz); cudaFreeHost(s.bucket); cudaFreeHost(s.score); cudaFreeHost(s.wdl); }
    for (int i = 0; i < 2; ++i) {
        cudaFree(t->pre[i]); cudaFree(t->dft[i]);
        if (t->ev_upload[i]) cudaEventDestroy(t->ev_upload[i]);
        if (t->ev_consumed[i]) cudaEventDestroy(t->ev_consumed[i]);
        if (t->ev_loss[i]) cudaEventDestroy(t->ev_loss[i]);
        cudaFreeHost(t->loss_pinned[i]);
    }
    cudaFree(t->combined); cudaFree(t->l1_out); cudaFree(t->dl1); cudaFree(t->net_output); cudaFree(t->dy);
    cudaFree(t->tail_a); cudaFree(t->tail_b); cudaFree(t->tail_c); cudaFree(t->loss_partials); cudaFree(t->loss_acc); cudaFree(t->wrm_weight_sum);
    cudaFree(t->order); cudaFree(t->n_tiles); cudaFree(t->seg_start); cudaFree(t->tiles);
    cudaFree(t->small_partials); cudaFree(t->l1w_partials); cudaFree(t->bias_partials); cudaFree(t->l1_weff);
    cudaFree(t->feat_counts); cudaFree(t->feat_offsets); cudaFree(t->feat_cursor); cudaFree(t->feat_lists);
    cudaFree(t->fwd_work); cudaFree(t->bwd_slice); cudaFree(t->sort_hist); cudaFree(t->items); cudaFree(t->item_seg); cudaFree(t->bwd_plan); cudaFree(t->bwd_partial); cudaFree(t->bwd_slabs);
    if (t->ev_t0) cudaEventDestroy(t->ev_t0);
    if (t->ev_t1) cudaEventDestroy(t->ev_t1);
    for (int i = 0; i < PH_COUNT; ++i) {
        if (t->ph_start[i]) cudaEventDestroy(t->ph_start[i]);
        if (t->ph_stop[i]) cudaEventDestroy(t->ph_stop[i]);
    }
    if (t->comm_stream) cudaStreamDestroy(t->comm_stream);
    if (t->opt_stream) cudaStreamDestroy(t->opt_stream);
    for (auto& e : t->ev_part) if (e) cudaEventDestroy(e);
    for (auto& e : t->ev_reduced) if (e) cudaEventDestroy(e);
    if (t->ev_opt_done) cudaEventDestroy(t->ev_opt_done);
    if (t->ev_comm_done) cudaEventDestroy(t->ev_comm_done);
    if (t->copy_stream) cudaStreamDestroy(t->copy_stream);
    if (t->stream) cudaStreamDestroy(t->stream);
    delete t;
}

int alloc_batch(tb_trainer* t, DevBatch* d) {
    const size_t B = (size_t)t->cfg.batch_capacity, A = (size_t)t->cfg.max_active;
    CU(t, dalloc(&d->stm, B * A)); CU(t, dalloc(&d->nstm, B * A)); CU(t, dalloc(&d->nnz, B)); CU(t, dalloc(&d->bucket, B));
    CU(t, dalloc(&d->score, B)); CU(t, dalloc(&d->wdl, B));
    return TB_OK;
}

int create_impl(tb_trainer* t) {
    const tb_config& c = t->cfg;
    CU(t, cudaSetDevice(c.device));
    CU(t, cudaDeviceGetAttribute(&t->n_sm, cudaDevAttrMultiProcessorCount, c.device));
    {
        // Data parallel: the step's own kernels go before the FT row updates that run behind the exchanged gradient parts
        // (opt_stream, lowest priority).  Both want whole SMs (the weight gradient holds all registers of its SM), so
        // running them side by side gains nothing; deferring the row updates fills the wave tails of the gradient parts
        // and the time the last part's exchange is in flight.
        int lo = 0, hi = 0;
        CU(t, cudaDeviceGetStreamPriorityRange(&lo, &hi));
        const int mid = c.world_size > 1 && hi < lo ? lo - 1 : lo;
        CU(t, cudaStreamCreateWithPriority(&t->stream, cudaStreamNonBlocking, mid));
    }
    CU(t, cudaStreamCreateWithFlags(&t->copy_stream, cudaStreamNonBlocking));
    const bool ls = c.arch == TB_ARCH_LAYERSTACK;
    const int64_t N = c.ft_in, F = c.ft_out, l1 = c.l1_out, l2 = c.l2_out, nb = c.num_buckets;
    t->p_tf32 = (c.precision & TB_PREC_TF32) != 0;
    t->p_ft16 = (c.precision & TB_PREC_FT_FP16) != 0;
    t->p_out16 = (c.precision & TB_PREC_FT_FP16_OUT) != 0;
    t->p_state16 = (c.precision & TB_PREC_FP16_OPT_STATE) != 0;
    t->Nt = c.ft_in + (c.ft_factorize ? c.piece_inputs : 0);
    t->l1e = c.l1_out - 1;
    t->l2in = 2 * t->l1e;
    t->K = (ls || c.activation == TB_ACT_PAIRWISE) ? c.ft_out : 2 * c.ft_out;  // width of the L1 input
    auto add = [&](const char* name, int kind, float clamp, int64_t len) {
        Group g; g.name = name; g.kind = kind; g.clamp = clamp; g.len = len; t->groups.push_back(g);
    };
    // group tables: trainer_layerstack.rs:740-762, trainer_simple.rs:2497-2578
    add("ft_w", 0, CLAMP_NONE, (int64_t)t->Nt * F);
    add("ft_b", 2, CLAMP_NONE, F);
    if (ls) {
        add("l1_w", 1, CLAMP_Q, nb * l1 * F);
        add("l1_b", 2, CLAMP_Q, nb * l1);
        add("l1_shared_weight", 1, CLAMP_Q, F * l1);
        add("l1_shared_bias", 2, CLAMP_Q, l1);
        add("l2_w", 1, CLAMP_Q, nb * l2 * t->l2in);
        add("l2_b", 2, CLAMP_Q, nb * l2);
        add("l3_w", 1, CLAMP_Q, nb * l2);
        add("l3_b", 2, CLAMP_NONE, nb);
    } else {
        add("l1_w", 1, CLAMP_Q, (int64_t)t->K * l1);
        add("l1_b", 2, CLAMP_Q, l1);
        add("l2_w", 1, CLAMP_Q, l1 * l2);
        add("l2_b", 2, CLAMP_Q, l2);
        add("l3_w", 1, CLAMP_Q, l2);
        add("l3_b", 2, CLAMP_NONE, 1);
    }
    // gradient arena: small groups first, then the real FT rows, then the virtual FT rows (which are derived
    // from the real rows after the all-reduce and therefore stay out of it)
    int64_t off = 0;
    std::vector<int64_t> goff(t->groups.size());
    for (size_t i = 1; i < t->groups.size(); ++i) { goff[i] = off; off += (t->groups[i].len + 3) / 4 * 4; }
    goff[0] = off;
    t->arena_reduce_len = off + N * F;
    t->arena_len = off + t->groups[0].len;
    CU(t, dalloc(&t->grad_arena, (size_t)t->arena_len));
    for (size_t i = 0; i < t->groups.size(); ++i) {
        Group& g = t->groups[i];
        g.grad = t->grad_arena + goff[i];
        CU(t, dalloc(&g.w, (size_t)g.len));
        if (i == 0 && t->p_state16) {  // MomentBuf::F16 (trainer_common.rs:60-71): only the FT table's moments
            CU(t, dalloc((__half**)&t->ft_m_h, (size_t)g.len)); CU(t, dalloc((__half**)&t->ft_v_h, (size_t)g.len));
        } else {
            CU(t, dalloc(&g.m, (size_t)g.len)); CU(t, dalloc(&g.v, (size_t)g.len));
        }
        CU(t, dalloc(&g.slow, (size_t)(c.optimizer == TB_OPT_RANGER ? g.len : 1)));
    }
    // the table the forward reads: fp32 folded table, or one fp16 table (folded, or the mirror of the master rows)
    if (t->p_ft16) CU(t, dalloc((__half**)&t->table_h, (size_t)(N * F)));
    else if (c.ft_factorize) CU(t, dalloc(&t->comb, (size_t)(N * F)));
    if (t->p_out16) CU(t, dalloc(&t->clamp_counter, 1));
    if (t->p_tf32) {
        CU(t, dalloc(&t->tc_error, 1));
        CU(t, cudaHostAlloc((void**)&t->tc_error_pinned, sizeof(int), cudaHostAllocDefault));
        *t->tc_error_pinned = 0;
    }

    const size_t B = (size_t)c.batch_capacity, A = (size_t)c.max_active;
    for (auto& d : t->ring) { int rc = alloc_batch(t, &d); if (rc) return rc; }
    for (auto& d : t->slots) { int rc = alloc_batch(t, &d); if (rc) return rc; }
    for (auto& s : t->stage) {
        CU(t, cudaHostAlloc((void**)&s.stm, B * A * 4, cudaHostAllocDefault)); CU(t, cudaHostAlloc((void**)&s.nstm, B * A * 4, cudaHostAllocDefault));
        CU(t, cudaHostAlloc((void**)&s.nnz, B * 4, cudaHostAllocDefault)); CU(t, cudaHostAlloc((void**)&s.bucket, B * 4, cudaHostAllocDefault));
        CU(t, cudaHostAlloc((void**)&s.score, B * 4, cudaHostAllocDefault)); CU(t, cudaHostAlloc((void**)&s.wdl, B * 4, cudaHostAllocDefault));
    }
    for (int i = 0; i < 2; ++i) {
        CU(t, dalloc(&t->ring_psv[i], B * 40));
        CU(t, cudaHostAlloc((void**)&t->stage_psv[i], B * 40, cudaHostAllocDefault));
        CU(t, cudaEventCreateWithFlags(&t->ev_upload[i], cudaEventDisableTiming));
        CU(t, cudaEventCreateWithFlags(&t->ev_consumed[i], cudaEventDisableTiming));
        CU(t, cudaEventCreateWithFlags(&t->ev_loss[i], cudaEventDisableTiming));
        CU(t, cudaHostAlloc((void**)&t->loss_pinned[i], sizeof(double), cudaHostAllocDefault));
        *t->loss_pinned[i] = 0.0;
        if (t->p_out16) {
            CU(t, dalloc((__half**)&t->pre_h[i], B * F));
            CU(t, dalloc((__half**)&t->dft_h[i], B * F));
        } else {
            CU(t, dalloc(&t->pre[i], B * F));
            CU(t, dalloc(&t->dft[i], B * F));
        }
    }
    CU(t, dalloc(&t->combined, B * (size_t)t->K));
    CU(t, dalloc(&t->l1_out, B * l1)); CU(t, dalloc(&t->dl1, B * l1));
    CU(t, dalloc(&t->net_output, B)); CU(t, dalloc(&t->dy, B));
    CU(t, dalloc(&t->tail_a, B * (size_t)(ls ? t->l2in : l1)));
    CU(t, dalloc(&t->tail_b, B * l2)); CU(t, dalloc(&t->tail_c, B * l2));
    CU(t, dalloc(&t->loss_partials, B / 128 + 1024)); CU(t, dalloc(&t->loss_acc, 1));  // one partial per tail block (<= 148 * 4 or B / 128)
    CU(t, dalloc(&t->wrm_weight_sum, 1));
    t->max_tiles = (int)(B / TB_TILE_M) + TB_MAX_BUCKETS + 2;
    t->max_units = sort_max_units(t->max_tiles);
    CU(t, dalloc(&t->order, B)); CU(t, dalloc(&t->n_tiles, 2)); CU(t, dalloc(&t->seg_start, TB_MAX_BUCKETS + 3));
    CU(t, dalloc(&t->tiles, (size_t)t->max_tiles + t->max_units));
    const size_t n_cells = ls ? (size_t)(l2 * t->l2in + 2 * l2 + 1 + l1) : (size_t)(l1 * l2 + 2 * l2 + 1 + l1);
    CU(t, dalloc(&t->small_partials, (ls ? (size_t)(nb + 1) * 64 : (size_t)128) * n_cells));  // SW_SPLIT_LS partial rows per segment
    CU(t, dalloc(&t->l1w_partials, ((size_t)t->max_units + 1) * l1 * t->K));
    CU(t, dalloc(&t->l1_weff, (size_t)(nb + 1) * l1 * (t->K + 1)));  // effective L1 weights and biases per bucket
    t->dgrad_rows = DGRAD_CTAS > 2 * t->max_units ? DGRAD_CTAS : 2 * t->max_units;  // partial FT bias rows: one per block
    CU(t, dalloc(&t->bias_partials, (size_t)t->dgrad_rows * 2 * F));
    CU(t, dalloc(&t->feat_counts, inverse_index_counts_len((int)N))); CU(t, dalloc(&t->feat_offsets, (size_t)2 * (N + 1)));
    // histograms of the item sort and of the bucket sort
    CU(t, dalloc(&t->sort_hist, (size_t)128 * (2 * B / 1024 + 2) + (size_t)(TB_MAX_BUCKETS + 1) * (B / 1024 + 2)));
    CU(t, dalloc(&t->items, 2 * B)); CU(t, dalloc(&t->item_seg, 130));
    CU(t, dalloc(&t->fwd_work, ft_forward_slice_work_ints((int)(2 * B), 129, A)));
    {
        const int rps = c.piece_inputs > 0 ? c.piece_inputs : (int)N;
        if (ft_forward_slice_supported((int)F, (int)N, (int)A, rps) && ft_backward_slice_supported((int)F, (int)N, (int)A, rps))
        {
            CU(t, dalloc(&t->bwd_slice, ft_backward_slice_ints((int)(2 * B), (int)A, rps)));
            CU(t, cudaMalloc((void**)&t->bwd_slabs, ft_backward_slice_slab_floats((int)(2 * B), (int)A, rps, (int)F) * sizeof(float)));
        }
    }
    {
        const size_t max_work = (size_t)ft_backward_max_work((int)B, (int)A, 2);
        CU(t, dalloc(&t->bwd_plan, 2 + 2 * max_work + 3 * (size_t)N));
        CU(t, dalloc(&t->bwd_partial, max_work * (size_t)F));
    }
    CU(t, dalloc(&t->feat_cursor, (size_t)2 * N)); CU(t, dalloc(&t->feat_lists, (size_t)4 * B * A));
    CU(t, cudaEventCreate(&t->ev_t0)); CU(t, cudaEventCreate(&t->ev_t1));
    for (int i = 0; i < PH_COUNT; ++i) {
        CU(t, cudaEventCreate(&t->ph_start[i])); CU(t, cudaEventCreate(&t->ph_stop[i]));
    }
    if (c.world_size > 1) {
        std::string e;
        if (!load_nccl(&e)) return fail(t, TB_ERR_NCCL, "%s", e.c_str());
        Uid id;
        memcpy(id.internal, c.nccl_unique_id, 128);
        int rc;
        if (c.nccl_ctas > 0) {
            // ncclConfig_t as NCCL 2.17 declares it (later versions only append fields, and the library reads `size` bytes
            // and takes its defaults for the rest): a fixed number of CTAs = channels for this communicator alone
            struct { size_t size; unsigned magic, version; int blocking, cga_cluster_size, min_ctas, max_ctas; const char* net_name; } nc;
            nc.size = sizeof(nc); nc.magic = 0xcafebeefu; nc.version = 21700;
            nc.blocking = INT_MIN; nc.cga_cluster_size = INT_MIN; nc.min_ctas = nc.max_ctas = c.nccl_ctas; nc.net_name = nullptr;
            rc = g_nccl.CommInitRankConfig(&t->comm, c.world_size, id, c.rank, &nc);
        } else {
            rc = g_nccl.CommInitRank(&t->comm, c.world_size, id, c.rank);
        }
        if (rc != 0) return fail(t, TB_ERR_NCCL, "ncclCommInitRank%s: %s", c.nccl_ctas > 0 ? "Config" : "", g_nccl.GetErrorString(rc));
        if (c.dp_exchange == TB_DP_PEER_COPY || c.dp_exchange == TB_DP_PEER_KERNEL) {
            std::string e2;
            if (px_create(&t->px, c.dp_exchange == TB_DP_PEER_COPY ? PX_MODE_COPY : PX_MODE_KERNEL, c.rank, c.world_size, t->grad_arena, (size_t)t->arena_reduce_len, AR_PARTS_MAX, t->loss_acc,
                          nccl_host_allgather, t, &e2) != 0)
                return fail(t, TB_ERR_CUDA, "%s", e2.c_str());
        }
        {   // highest priority: when an SM frees up, the waiting all-reduce gets it before the next gradient block does
            int lo = 0, hi = 0;
            CU(t, cudaDeviceGetStreamPriorityRange(&lo, &hi));
            CU(t, cudaStreamCreateWithPriority(&t->comm_stream, cudaStreamNonBlocking, hi));
        }
        CU(t, cudaStreamCreateWithFlags(&t->opt_stream, cudaStreamNonBlocking));
        for (auto& e : t->ev_part) CU(t, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        for (auto& e : t->ev_reduced) CU(t, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        CU(t, cudaEventCreateWithFlags(&t->ev_opt_done, cudaEventDisableTiming));
        CU(t, cudaEventCreateWithFlags(&t->ev_comm_done, cudaEventDisableTiming));
        if (getenv("TATARA_DP_TRACE")) {
            t->dp_trace = true;
            CU(t, cudaEventCreate(&t->tr_start)); CU(t, cudaEventCreate(&t->tr_done));
            for (int i = 0; i < AR_PARTS_MAX; ++i) {
                CU(t, cudaEventCreate(&t->tr_part[i])); CU(t, cudaEventCreate(&t->tr_red[i]));
                CU(t, cudaEventCreate(&t->tr_opt0[i])); CU(t, cudaEventCreate(&t->tr_opt1[i]));
            }
        }
    }
    CU(t, cudaDeviceSynchronize());
    return TB_OK;
}

int validate_config(const tb_config* c) {
    if (!c) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "config is NULL");
    if (c->struct_size != (int32_t)sizeof(tb_config))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "tb_config.struct_size %d != %d (header / library mismatch)", c->struct_size, (int)sizeof(tb_config));
    if (c->arch != TB_ARCH_LAYERSTACK && c->arch != TB_ARCH_SIMPLE) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "unknown arch %d", c->arch);
    if (c->batch_capacity < 16 || c->batch_capacity % 16 != 0 || c->batch_capacity > (1 << 20))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "batch_capacity must be a multiple of 16 in [16, 2^20] (got %d)", c->batch_capacity);
    if (c->ft_out < 128 || c->ft_out % 128 != 0 || c->ft_out > 4096)
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "ft_out must be a multiple of 128 in [128, 4096] (got %d)", c->ft_out);
    if (c->arch == TB_ARCH_SIMPLE && (c->activation < TB_ACT_CRELU || c->activation > TB_ACT_PAIRWISE))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "unknown activation %d", c->activation);
    if ((c->arch == TB_ARCH_LAYERSTACK || c->activation == TB_ACT_PAIRWISE) && c->ft_out < 256)
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "the pairwise FT activation needs ft_out >= 256 (got %d)", c->ft_out);
    if (false)
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "LayerStack needs ft_out >= 256 (got %d)", c->ft_out);
    if (c->ft_in < 1 || c->max_active < 1 || c->max_active > 256) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "bad ft_in / max_active");
    if (c->ft_factorize && (c->piece_inputs < 1 || c->ft_in % c->piece_inputs != 0))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "ft_factorize needs ft_in (%d) divisible by piece_inputs (%d)", c->ft_in, c->piece_inputs);
    if (c->l1_out < 2 || c->l1_out > TB_MAX_L1) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "l1_out must be in [2, %d]", TB_MAX_L1);
    if (c->l2_out < 1 || c->l2_out > TB_MAX_L2) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "l2_out must be in [1, %d]", TB_MAX_L2);
    // trainer_layerstack.rs:797-800
    if (c->arch == TB_ARCH_LAYERSTACK && (c->num_buckets < 2 || c->num_buckets > TB_MAX_BUCKETS))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "LayerStack requires num_buckets in [2, %d]", TB_MAX_BUCKETS);
    if (c->optimizer < TB_OPT_RANGER || c->optimizer > TB_OPT_ADAMW) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "unknown optimizer %d", c->optimizer);
    // trainer_layerstack.rs:801-805
    if ((c->precision & TB_PREC_FT_FP16_OUT) && !(c->precision & TB_PREC_FT_FP16))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "--ft-fp16-out requires --ft-fp16");
    if (c->precision & ~(TB_PREC_TF32 | TB_PREC_FT_FP16 | TB_PREC_FT_FP16_OUT | TB_PREC_FP16_OPT_STATE))
        return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "unknown precision bits %#x", c->precision);
    if (c->precision != 0) {
        // What is built: the LayerStack trainer with l1_out of 8, 16 or 32 (the streaming L1 kernels) on a king-relative
        // feature set (the slice-resident FT kernels are the only ones with fp16 rows at speed; the generic kernels serve
        // batches that break the slice property).
        if (c->arch != TB_ARCH_LAYERSTACK)
            return fail(nullptr, TB_ERR_UNSUPPORTED, "reduced-precision modes are built for the LayerStack architecture only");
        if (c->l1_out != 8 && c->l1_out != 16 && c->l1_out != 32)
            return fail(nullptr, TB_ERR_UNSUPPORTED, "reduced-precision modes need l1_out of 8, 16 or 32 (got %d)", c->l1_out);
    }
    if (c->world_size < 1 || c->rank < 0 || c->rank >= c->world_size) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "bad rank %d / world_size %d", c->rank, c->world_size);
    return TB_OK;
}

}  // namespace

// ==================================================================================================
// C ABI
// ==================================================================================================
extern "C" {

int tb_create(const tb_config* cfg, tb_trainer** out) {
    if (!out) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "out is NULL");
    *out = nullptr;
    int rc = validate_config(cfg);
    if (rc != TB_OK) return rc;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev < 1) { cudaGetLastError(); return fail(nullptr, TB_ERR_NO_DEVICE, "no CUDA device is available"); }
    if (cfg->device < 0 || cfg->device >= n_dev) return fail(nullptr, TB_ERR_NO_DEVICE, "device %d out of range (%d devices)", cfg->device, n_dev);
    tb_trainer* t = new tb_trainer();
    t->cfg = *cfg;
    for (int i = 0; i < PH_COUNT; ++i) { t->ph_start[i] = t->ph_stop[i] = nullptr; t->ph_used[i] = false; t->ph_ms[i] = 0.0; t->ph_launches[i] = 0; }
    rc = create_impl(t);
    if (rc != TB_OK) { g_create_error = t->err; free_all(t); return rc; }
    *out = t;
    return TB_OK;
}

void tb_destroy(tb_trainer* t) {
    if (!t) return;
    cudaSetDevice(t->cfg.device);
    free_all(t);
}

const char* tb_last_error(const tb_trainer* t) { return t ? t->err.c_str() : g_create_error.c_str(); }

int tb_num_groups(const tb_trainer* t) { return t ? (int)t->groups.size() : 0; }
const char* tb_group_name(const tb_trainer* t, int g) { return (t && g >= 0 && g < (int)t->groups.size()) ? t->groups[g].name.c_str() : nullptr; }
int64_t tb_group_len(const tb_trainer* t, const char* name) {
    Group* g = find_group(const_cast<tb_trainer*>(t), name);
    return g ? g->len : -1;
}

int tb_upload_group(tb_trainer* t, const char* name, const float* w, const float* m, const float* v, const float* slow, int64_t len) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    Group* g = find_group(t, name);
    if (!g) return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown group '%s'", name ? name : "(null)");
    if (len != g->len) return fail(t, TB_ERR_INVALID_ARGUMENT, "group '%s' has %lld elements, got %lld", name, (long long)g->len, (long long)len);
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->stream));
    const size_t bytes = (size_t)len * 4;
    const bool ft = g == &t->groups[0];
    if (w) CU(t, cudaMemcpy(g->w, w, bytes, cudaMemcpyHostToDevice));
    if (ft && t->p_state16) {
        // MomentBuf::from_host_f32 (trainer_common.rs:107-126): true f32 moments are scaled, clamped to the fp16 range
        // and rounded
        std::vector<__half> h((size_t)len);
        const float* src[2] = {m, v};
        void* dst[2] = {t->ft_m_h, t->ft_v_h};
        const float scale[2] = {TB_FT_OPT_M_SCALE, TB_FT_OPT_V_SCALE};
        for (int k = 0; k < 2; ++k) {
            if (!src[k]) continue;
            for (int64_t i = 0; i < len; ++i) {
                float x = src[k][i] * scale[k];
                x = x > 65504.0f ? 65504.0f : (x < -65504.0f ? -65504.0f : x);
                h[(size_t)i] = __float2half_rn(x);
            }
            CU(t, cudaMemcpy(dst[k], h.data(), (size_t)len * 2, cudaMemcpyHostToDevice));
        }
    } else {
        if (m) CU(t, cudaMemcpy(g->m, m, bytes, cudaMemcpyHostToDevice));
        if (v) CU(t, cudaMemcpy(g->v, v, bytes, cudaMemcpyHostToDevice));
    }
    if (slow && t->cfg.optimizer == TB_OPT_RANGER) CU(t, cudaMemcpy(g->slow, slow, bytes, cudaMemcpyHostToDevice));
    if (w && ft && (t->cfg.ft_factorize || t->p_ft16)) {
        // sync_ft_forward_weights: the table the forward reads follows the master weights (fold, and / or fp16 cast)
        if (t->cfg.ft_factorize)
            t->launches += launch_ft_fold(t->stream, g->w, t->p_ft16 ? t->table_h : (void*)t->comb, t->cfg.ft_in, t->cfg.piece_inputs,
                                          t->cfg.ft_out, t->p_ft16);
        else
            t->launches += launch_cast_half(t->stream, g->w, t->table_h, g->len);
        CU(t, cudaStreamSynchronize(t->stream));
    }
    return TB_OK;
}

int tb_download_group(tb_trainer* t, const char* name, float* w, float* m, float* v, float* slow, int64_t len) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    Group* g = find_group(t, name);
    if (!g) return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown group '%s'", name ? name : "(null)");
    if (len != g->len) return fail(t, TB_ERR_INVALID_ARGUMENT, "group '%s' has %lld elements, got %lld", name, (long long)g->len, (long long)len);
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->stream));
    const size_t bytes = (size_t)len * 4;
    if (w) CU(t, cudaMemcpy(w, g->w, bytes, cudaMemcpyDeviceToHost));
    if (g == &t->groups[0] && t->p_state16) {
        // MomentBuf::to_host_f32 (trainer_common.rs:89-105): stored fp16 values divided by their scale
        std::vector<__half> h((size_t)len);
        float* dst[2] = {m, v};
        const void* src[2] = {t->ft_m_h, t->ft_v_h};
        const float inv[2] = {1.0f / TB_FT_OPT_M_SCALE, 1.0f / TB_FT_OPT_V_SCALE};
        for (int k = 0; k < 2; ++k) {
            if (!dst[k]) continue;
            CU(t, cudaMemcpy(h.data(), src[k], (size_t)len * 2, cudaMemcpyDeviceToHost));
            for (int64_t i = 0; i < len; ++i) dst[k][i] = __half2float(h[(size_t)i]) * inv[k];
        }
    } else {
        if (m) CU(t, cudaMemcpy(m, g->m, bytes, cudaMemcpyDeviceToHost));
        if (v) CU(t, cudaMemcpy(v, g->v, bytes, cudaMemcpyDeviceToHost));
    }
    if (slow) {
        if (t->cfg.optimizer == TB_OPT_RANGER) CU(t, cudaMemcpy(slow, g->slow, bytes, cudaMemcpyDeviceToHost));
        else memset(slow, 0, bytes);
    }
    return TB_OK;
}

int tb_get_step_count(const tb_trainer* t, uint64_t* s) { if (!t || !s) return TB_ERR_INVALID_ARGUMENT; *s = t->step_count; return TB_OK; }
int tb_set_step_count(tb_trainer* t, uint64_t s) { if (!t) return TB_ERR_INVALID_ARGUMENT; t->step_count = s; return TB_OK; }

int tb_train_step(tb_trainer* t, const tb_batch* batch, float lr, float wdl_lambda, const tb_loss* loss, double* loss_prev) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    int rc = check_batch(t, batch);
    if (rc == TB_OK) rc = check_loss(t, loss);
    if (rc != TB_OK) return rc;
    if (batch->n_pos == 0) { if (loss_prev) *loss_prev = 0.0; return TB_OK; }  // trainer_layerstack.rs:2018-2023
    CU(t, cudaSetDevice(t->cfg.device));
    int s = 0;
    rc = ring_upload(t, batch, &s);
    if (rc != TB_OK) return rc;
    rc = step_on(t, t->ring[s], lr, wdl_lambda, loss, loss_prev);
    if (rc != TB_OK) return rc;
    CU(t, cudaEventRecord(t->ev_consumed[s], t->stream));
    t->consumed_pending[s] = true;
    return TB_OK;
}

int tb_train_step_psv(tb_trainer* t, int feature_set, const uint8_t* psv, int n_pos, float lr, float wdl_lambda,
                      const tb_loss* loss, double* loss_prev) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    int rc = check_loss(t, loss);
    if (rc != TB_OK) return rc;
    if (n_pos < 0) return fail(t, TB_ERR_INVALID_ARGUMENT, "n_pos is negative (%d)", n_pos);
    if (n_pos == 0) { if (loss_prev) *loss_prev = 0.0; return TB_OK; }
    if (!psv) return fail(t, TB_ERR_INVALID_ARGUMENT, "psv is NULL");
    if (n_pos % 16 != 0) return fail(t, TB_ERR_INVALID_ARGUMENT, "n_pos must be a multiple of 16 (got %d)", n_pos);
    if (n_pos > t->cfg.batch_capacity)
        return fail(t, TB_ERR_INVALID_ARGUMENT, "batch %d exceeds workspace capacity %d (the workspace is allocated once at creation)",
                    n_pos, t->cfg.batch_capacity);
    int fs_in = 0, fs_active = 0;
    if (!psv_feature_set_dims(feature_set, &fs_in, &fs_active)) return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown feature set id %d", feature_set);
    // the batch's feature set must be the trainer's (bins/nnue_train/src/trainer_common.rs:301-307)
    if (fs_in != t->cfg.ft_in || fs_active != t->cfg.max_active)
        return fail(t, TB_ERR_INVALID_ARGUMENT, "feature set %d has ft_in %d / max_active %d, the trainer was created with %d / %d",
                    feature_set, fs_in, fs_active, t->cfg.ft_in, t->cfg.max_active);
    CU(t, cudaSetDevice(t->cfg.device));
    int s = 0;
    rc = ring_upload_psv(t, feature_set, psv, n_pos, &s);
    if (rc != TB_OK) return rc;
    rc = step_on(t, t->ring[s], lr, wdl_lambda, loss, loss_prev);
    if (rc != TB_OK) return rc;
    CU(t, cudaEventRecord(t->ev_consumed[s], t->stream));
    t->consumed_pending[s] = true;
    return TB_OK;
}

int tb_flush_pending_loss(tb_trainer* t, double* loss) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    double returned = 0.0;
    if (t->loss_primed) {
        const int last = (int)((t->loss_step + 1) % 2);
        { const int wrc = wait_loss_event(t, t->ev_loss[last]); if (wrc != TB_OK) return wrc; }
        returned = *t->loss_pinned[last];
    }
    t->loss_primed = false;
    t->loss_step = 0;
    if (loss) *loss = returned;
    return TB_OK;
}

int tb_validate_step(tb_trainer* t, const tb_batch* batch, float wdl_lambda, const tb_loss* loss, double* sum_sq_err, float* net_output) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    int rc = check_batch(t, batch);
    if (rc == TB_OK) rc = check_loss(t, loss);
    if (rc != TB_OK) return rc;
    if (batch->n_pos == 0) { if (sum_sq_err) *sum_sq_err = 0.0; return TB_OK; }
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->stream));  // GpuTrainer::validate drains the stream first
    DevBatch& d = t->slots[TB_NUM_SLOTS - 1];
    tb_batch b = *batch;
    if (b.per_pos_norm == 0.f) b.per_pos_norm = 1.0f / (float)b.n_pos;
    rc = upload_batch(t, &b, &d, nullptr, t->stream);
    if (rc != TB_OK) return rc;
    rc = run_forward(t, d, loss, wdl_lambda, 0);
    if (rc != TB_OK) return rc;
    double l = 0.0;
    CU(t, cudaMemcpyAsync(&l, t->loss_acc, sizeof(double), cudaMemcpyDeviceToHost, t->stream));
    if (net_output) CU(t, cudaMemcpyAsync(net_output, t->net_output, (size_t)b.n_pos * 4, cudaMemcpyDeviceToHost, t->stream));
    CU(t, cudaStreamSynchronize(t->stream));
    profile_collect(t);
    if (sum_sq_err) *sum_sq_err = l;
    return TB_OK;
}

int tb_read_fp16_clamp_count(tb_trainer* t, uint64_t* clamps, uint64_t* elems) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    // (clamped, written) dft elements so far, like GpuTrainer::read_fp16_clamp_count (crates/nnue-train/src/trainer.rs:1100-1119);
    // zeros unless the FT activations are fp16
    unsigned long long n = 0;
    if (t->p_out16) {
        CU(t, cudaSetDevice(t->cfg.device));
        CU(t, cudaStreamSynchronize(t->stream));
        CU(t, cudaMemcpy(&n, t->clamp_counter, sizeof n, cudaMemcpyDeviceToHost));
    }
    if (clamps) *clamps = n;
    if (elems) *elems = t->clamp_elems;
    return TB_OK;
}

int tb_stage_batch(tb_trainer* t, int slot, const tb_batch* batch) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    if (slot < 0 || slot >= TB_NUM_SLOTS - 1) return fail(t, TB_ERR_INVALID_ARGUMENT, "slot %d out of range [0, %d)", slot, TB_NUM_SLOTS - 1);
    int rc = check_batch(t, batch);
    if (rc != TB_OK) return rc;
    if (batch->n_pos == 0) return fail(t, TB_ERR_INVALID_ARGUMENT, "cannot stage an empty batch");
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->stream));
    rc = upload_batch(t, batch, &t->slots[slot], nullptr, t->stream);
    if (rc != TB_OK) return rc;
    CU(t, cudaStreamSynchronize(t->stream));
    return TB_OK;
}

int tb_train_step_staged(tb_trainer* t, int slot, float lr, float wdl_lambda, const tb_loss* loss, double* loss_prev) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    if (slot < 0 || slot >= TB_NUM_SLOTS - 1 || t->slots[slot].n_pos == 0) return fail(t, TB_ERR_INVALID_ARGUMENT, "slot %d holds no batch", slot);
    int rc = check_loss(t, loss);
    if (rc != TB_OK) return rc;
    CU(t, cudaSetDevice(t->cfg.device));
    return step_on(t, t->slots[slot], lr, wdl_lambda, loss, loss_prev);
}

int tb_forward_backward(tb_trainer* t, const tb_batch* batch, float wdl_lambda, const tb_loss* loss, double* loss_now) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    int rc = check_batch(t, batch);
    if (rc == TB_OK) rc = check_loss(t, loss);
    if (rc != TB_OK) return rc;
    if (batch->n_pos == 0) { if (loss_now) *loss_now = 0.0; return TB_OK; }
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->stream));
    DevBatch& d = t->slots[TB_NUM_SLOTS - 1];
    rc = upload_batch(t, batch, &d, nullptr, t->stream);
    if (rc == TB_OK) rc = run_forward(t, d, loss, wdl_lambda, 1);
    if (rc == TB_OK) rc = run_backward(t, d, -1.0f);
    if (rc == TB_OK) rc = run_allreduce(t);
    if (rc != TB_OK) return rc;
    if (t->cfg.ft_factorize)
        t->launches += launch_ft_reduce_virtual(t->stream, t->groups[0].grad, t->cfg.ft_in, t->cfg.piece_inputs, t->cfg.ft_out);
    double l = 0.0;
    CU(t, cudaMemcpyAsync(&l, t->loss_acc, sizeof(double), cudaMemcpyDeviceToHost, t->stream));
    if (t->tc_error) CU(t, cudaMemcpyAsync(t->tc_error_pinned, t->tc_error, sizeof(int), cudaMemcpyDeviceToHost, t->stream));
    CU(t, cudaStreamSynchronize(t->stream));
    CU(t, cudaGetLastError());
    profile_collect(t);
    if (t->tc_error && *t->tc_error_pinned) return fail(t, TB_ERR_CUDA, "the tensor-core L1 kernel gave up waiting for its MMAs");
    if (loss_now) *loss_now = l;
    return TB_OK;
}

int tb_apply_optimizer(tb_trainer* t, float lr) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    CU(t, cudaSetDevice(t->cfg.device));
    int rc = run_optimizer(t, lr);
    if (rc != TB_OK) return rc;
    CU(t, cudaStreamSynchronize(t->stream));
    CU(t, cudaGetLastError());
    profile_collect(t);
    return TB_OK;
}

int tb_download_grad(tb_trainer* t, const char* name, float* grad, int64_t len) {
    if (!t || !grad) return TB_ERR_INVALID_ARGUMENT;
    Group* g = find_group(t, name);
    if (!g) return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown group '%s'", name ? name : "(null)");
    if (len != g->len) return fail(t, TB_ERR_INVALID_ARGUMENT, "group '%s' has %lld elements, got %lld", name, (long long)g->len, (long long)len);
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->stream));
    CU(t, cudaMemcpy(grad, g->grad, (size_t)len * 4, cudaMemcpyDeviceToHost));
    // summed from loss-scaled fp16 rows: the rows still carry that scale (the optimizer takes it out on load)
    if (g == &t->groups[0] && t->p_out16)
        for (int64_t i = 0; i < len; ++i) grad[i] *= t->grad_unscale;
    return TB_OK;
}

int tb_read_buffer(tb_trainer* t, const char* name, float* out, int64_t len) {
    if (!t || !name || !out) return TB_ERR_INVALID_ARGUMENT;
    const tb_config& c = t->cfg;
    const int64_t B = t->last_n, F = c.ft_out;
    // fp16 buffers are returned as fp32 values; the fp16 dft rows with their loss scale taken out
    const bool o16 = t->p_out16, t16 = t->p_ft16;
    struct { const char* n; const void* p; int64_t l; bool half; float mul; } tab[] = {
        {"ft_stm", o16 ? t->pre_h[0] : (void*)t->pre[0], B * F, o16, 1.f}, {"ft_nstm", o16 ? t->pre_h[1] : (void*)t->pre[1], B * F, o16, 1.f},
        {"combined", t->combined, B * t->K, false, 1.f}, {"l1_total", t->l1_out, B * c.l1_out, false, 1.f},
        {"net_output", t->net_output, B, false, 1.f}, {"dy", t->dy, B, false, 1.f}, {"dl1_total", t->dl1, B * c.l1_out, false, 1.f},
        {"dft_stm", o16 ? t->dft_h[0] : (void*)t->dft[0], B * F, o16, o16 ? t->grad_unscale : 1.f},
        {"dft_nstm", o16 ? t->dft_h[1] : (void*)t->dft[1], B * F, o16, o16 ? t->grad_unscale : 1.f},
        {"comb", t16 ? t->table_h : (void*)t->comb, (t16 || t->comb) ? (int64_t)c.ft_in * F : 0, t16, 1.f}};
    for (auto& e : tab)
        if (strcmp(e.n, name) == 0) {
            if (len != e.l) return fail(t, TB_ERR_INVALID_ARGUMENT, "buffer '%s' has %lld elements, got %lld", name, (long long)e.l, (long long)len);
            CU(t, cudaSetDevice(c.device));
            CU(t, cudaStreamSynchronize(t->stream));
            if (len > 0 && !e.half) CU(t, cudaMemcpy(out, e.p, (size_t)len * 4, cudaMemcpyDeviceToHost));
            if (len > 0 && e.half) {
                std::vector<__half> h((size_t)len);
                CU(t, cudaMemcpy(h.data(), e.p, (size_t)len * 2, cudaMemcpyDeviceToHost));
                for (int64_t i = 0; i < len; ++i) out[i] = __half2float(h[(size_t)i]) * e.mul;
            }
            return TB_OK;
        }
    return fail(t, TB_ERR_INVALID_ARGUMENT, "unknown buffer '%s'", name);
}

int tb_timer_start(tb_trainer* t) { if (!t) return TB_ERR_INVALID_ARGUMENT; CU(t, cudaEventRecord(t->ev_t0, t->stream)); return TB_OK; }
int tb_timer_stop(tb_trainer* t, float* ms) {
    if (!t || !ms) return TB_ERR_INVALID_ARGUMENT;
    CU(t, cudaEventRecord(t->ev_t1, t->stream));
    CU(t, cudaEventSynchronize(t->ev_t1));
    CU(t, cudaEventElapsedTime(ms, t->ev_t0, t->ev_t1));
    return TB_OK;
}
int tb_profile_enable(tb_trainer* t, int on) { if (!t) return TB_ERR_INVALID_ARGUMENT; t->profile = on != 0; return TB_OK; }
int tb_profile_num_phases(const tb_trainer* t) { (void)t; return PH_COUNT; }
int tb_profile_read(tb_trainer* t, int phase, const char** name, double* total_ms, int64_t* launches) {
    if (!t || phase < 0 || phase >= PH_COUNT) return TB_ERR_INVALID_ARGUMENT;
    if (name) *name = kPhaseNames[phase];
    if (total_ms) *total_ms = t->ph_ms[phase];
    if (launches) *launches = t->ph_launches[phase];
    return TB_OK;
}
int tb_profile_reset(tb_trainer* t) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < PH_COUNT; ++i) { t->ph_ms[i] = 0.0; t->ph_launches[i] = 0; t->ph_used[i] = false; }
    return TB_OK;
}
int64_t tb_launch_count(const tb_trainer* t) { return t ? t->launches : 0; }
int tb_synchronize(tb_trainer* t) {
    if (!t) return TB_ERR_INVALID_ARGUMENT;
    CU(t, cudaSetDevice(t->cfg.device));
    CU(t, cudaStreamSynchronize(t->copy_stream));
    CU(t, cudaStreamSynchronize(t->stream));
    return TB_OK;
}

int tb_nccl_unique_id(uint8_t out[128]) {
    if (!out) return TB_ERR_INVALID_ARGUMENT;
    std::string e;
    if (!load_nccl(&e)) return fail(nullptr, TB_ERR_NCCL, "%s", e.c_str());
    Uid id;
    const int rc = g_nccl.GetUniqueId(&id);
    if (rc != 0) return fail(nullptr, TB_ERR_NCCL, "ncclGetUniqueId: %s", g_nccl.GetErrorString(rc));
    memcpy(out, id.internal, 128);
    return TB_OK;
}

int tb_host_alloc(void** out, size_t bytes) {
    if (!out) return TB_ERR_INVALID_ARGUMENT;
    cudaError_t e = cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault);
    if (e != cudaSuccess) { cudaGetLastError(); return fail(nullptr, TB_ERR_OUT_OF_MEMORY, "cudaHostAlloc(%zu): %s", bytes, cudaGetErrorString(e)); }
    return TB_OK;
}
int tb_host_free(void* p) {
    if (p && cudaFreeHost(p) != cudaSuccess) { cudaGetLastError(); return TB_ERR_CUDA; }
    return TB_OK;
}

int tb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

const char* tb_version(void) { return "tatara_b200 0.1 (sm_100a)"; }

// ---- FT kernels alone -------------------------------------------------------------------------------------
#define CUX(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { rc = fail(nullptr, TB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); goto done; } } while (0)

int tb_ft_forward_bench(int device, const float* table, const int32_t* indices, const int32_t* nnz, int batch, int ft_out,
                        int ft_in, int max_active, int iters, float* out, float* ms_per_iter) {
    if (!table || !indices || !nnz || batch < 1 || ft_out % 128 != 0 || iters < 1) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "bad argument");
    int rc = TB_OK;
    float *d_t = nullptr, *d_o = nullptr;
    int *d_i = nullptr, *d_n = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    const size_t B = batch, F = ft_out, N = ft_in, A = max_active;
    CUX(cudaSetDevice(device));
    CUX(cudaMalloc(&d_t, N * F * 4)); CUX(cudaMalloc(&d_o, B * F * 4)); CUX(cudaMalloc(&d_i, B * A * 4)); CUX(cudaMalloc(&d_n, B * 4));
    CUX(cudaMemcpy(d_t, table, N * F * 4, cudaMemcpyHostToDevice));
    CUX(cudaMemcpy(d_i, indices, B * A * 4, cudaMemcpyHostToDevice));
    CUX(cudaMemcpy(d_n, nnz, B * 4, cudaMemcpyHostToDevice));
    CUX(cudaEventCreate(&e0)); CUX(cudaEventCreate(&e1));
    launch_ft_forward(0, 0, d_t, d_i, d_i, d_n, nullptr, d_o, d_o, nullptr, nullptr, batch, ft_out, ft_in, max_active, 1.f, 1);
    CUX(cudaDeviceSynchronize());
    CUX(cudaEventRecord(e0, 0));
    for (int i = 0; i < iters; ++i) launch_ft_forward(0, 0, d_t, d_i, d_i, d_n, nullptr, d_o, d_o, nullptr, nullptr, batch, ft_out, ft_in, max_active, 1.f, 1);
    CUX(cudaEventRecord(e1, 0));
    CUX(cudaEventSynchronize(e1));
    { float ms = 0.f; CUX(cudaEventElapsedTime(&ms, e0, e1)); if (ms_per_iter) *ms_per_iter = ms / iters; }
    if (out) CUX(cudaMemcpy(out, d_o, B * F * 4, cudaMemcpyDeviceToHost));
done:
    cudaFree(d_t); cudaFree(d_o); cudaFree(d_i); cudaFree(d_n);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    return rc;
}

int tb_ft_backward_bench(int device, const float* dft, const int32_t* indices, const int32_t* nnz, int batch, int ft_out,
                         int ft_in, int max_active, int iters, float* grad, float* ms_per_iter) {
    if (!dft || !indices || !nnz || batch < 1 || ft_out % 128 != 0 || iters < 1) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "bad argument");
    int rc = TB_OK;
    float *d_d = nullptr, *d_g = nullptr;
    int *d_i = nullptr, *d_n = nullptr, *d_cnt = nullptr, *d_off = nullptr, *d_cur = nullptr, *d_lists = nullptr, *d_plan = nullptr;
    float* d_part = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    const size_t B = batch, F = ft_out, N = ft_in, A = max_active;
    const size_t max_work = (size_t)ft_backward_max_work(batch, max_active, 1);
    CUX(cudaSetDevice(device));
    CUX(cudaMalloc(&d_d, B * F * 4)); CUX(cudaMalloc(&d_g, N * F * 4)); CUX(cudaMalloc(&d_i, B * A * 4)); CUX(cudaMalloc(&d_n, B * 4));
    CUX(cudaMalloc(&d_cnt, inverse_index_counts_len(ft_in) * 4)); CUX(cudaMalloc(&d_off, 2 * (N + 1) * 4)); CUX(cudaMalloc(&d_cur, 2 * N * 4));
    CUX(cudaMalloc(&d_lists, 4 * B * A * 4));
    CUX(cudaMalloc(&d_plan, (2 + 2 * max_work + 3 * N) * 4)); CUX(cudaMalloc(&d_part, max_work * F * 4));
    CUX(cudaMemcpy(d_d, dft, B * F * 4, cudaMemcpyHostToDevice));
    CUX(cudaMemcpy(d_i, indices, B * A * 4, cudaMemcpyHostToDevice));
    CUX(cudaMemcpy(d_n, nnz, B * 4, cudaMemcpyHostToDevice));
    CUX(cudaEventCreate(&e0)); CUX(cudaEventCreate(&e1));
    for (int i = -1; i < iters; ++i) {
        if (i == 0) { CUX(cudaDeviceSynchronize()); CUX(cudaEventRecord(e0, 0)); }
        launch_inverse_index(0, nullptr, d_i, d_i, d_n, batch, max_active, ft_in, 1, d_cnt, d_off, d_cur, d_lists);
        launch_ft_backward_split(0, nullptr, d_d, d_d, d_off, d_lists, batch, max_active, ft_in, ft_out, 1, d_plan, d_part, d_g);
    }
    CUX(cudaEventRecord(e1, 0));
    CUX(cudaEventSynchronize(e1));
    { float ms = 0.f; CUX(cudaEventElapsedTime(&ms, e0, e1)); if (ms_per_iter) *ms_per_iter = ms / iters; }
    if (grad) CUX(cudaMemcpy(grad, d_g, N * F * 4, cudaMemcpyDeviceToHost));
done:
    cudaFree(d_d); cudaFree(d_g); cudaFree(d_i); cudaFree(d_n); cudaFree(d_cnt); cudaFree(d_off); cudaFree(d_cur); cudaFree(d_lists);
    cudaFree(d_plan); cudaFree(d_part);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    return rc;
}

int tb_adam_clamp_bench(int device, float* w, float* m, float* v, const float* grad, int64_t n, float lr, float decay,
                        float min_w, float max_w, int iters, float* ms_per_iter) {
    if (!w || !m || !v || !grad || n < 4 || n % 4 != 0 || iters < 1) return fail(nullptr, TB_ERR_INVALID_ARGUMENT, "bad argument");
    int rc = TB_OK;
    float *d_w = nullptr, *d_m = nullptr, *d_v = nullptr, *d_g = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    OptScalars sc;
    sc.lr = lr; sc.step_size = 1.f; sc.decay = decay; sc.beta1 = 0.9f; sc.beta2 = BETA2; sc.eps = EPS; sc.min_w = min_w; sc.max_w = max_w;
    sc.alpha = RANGER_ALPHA; sc.denom = 1; sc.lerp = 0;
    const size_t bytes = (size_t)n * 4;
    CUX(cudaSetDevice(device));
    CUX(cudaMalloc(&d_w, bytes)); CUX(cudaMalloc(&d_m, bytes)); CUX(cudaMalloc(&d_v, bytes)); CUX(cudaMalloc(&d_g, bytes));
    CUX(cudaMemcpy(d_w, w, bytes, cudaMemcpyHostToDevice)); CUX(cudaMemcpy(d_m, m, bytes, cudaMemcpyHostToDevice));
    CUX(cudaMemcpy(d_v, v, bytes, cudaMemcpyHostToDevice)); CUX(cudaMemcpy(d_g, grad, bytes, cudaMemcpyHostToDevice));
    CUX(cudaEventCreate(&e0)); CUX(cudaEventCreate(&e1));
    CUX(cudaEventRecord(e0, 0));
    for (int i = 0; i < iters; ++i) launch_radam(0, d_w, d_m, d_v, d_g, nullptr, n, sc);
    CUX(cudaEventRecord(e1, 0));
    CUX(cudaEventSynchronize(e1));
    { float ms = 0.f; CUX(cudaEventElapsedTime(&ms, e0, e1)); if (ms_per_iter) *ms_per_iter = ms / iters; }
    CUX(cudaMemcpy(w, d_w, bytes, cudaMemcpyDeviceToHost)); CUX(cudaMemcpy(m, d_m, bytes, cudaMemcpyDeviceToHost));
    CUX(cudaMemcpy(v, d_v, bytes, cudaMemcpyDeviceToHost));
done:
    cudaFree(d_w); cudaFree(d_m); cudaFree(d_v); cudaFree(d_g);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    return rc;
}

}  // extern "C"
