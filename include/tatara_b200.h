/*
 * tatara_b200 — C ABI of the sm_100a NNUE training step.
 *
 * The library replaces the device side of tatara's trainer backends.  One handle
 * corresponds to one `GpuTrainer` (LayerStack) or `SimpleGpuTrainer` (Simple) of the
 * reference; the entry points below are what an `impl TrainerBackend` over FFI binds.
 * Paths in the comments are relative to the reference project root.
 *
 * Conventions (the reference's, kept):
 *  - every call returns TB_OK or a negative error code; nothing aborts.  The text of
 *    the last error is available from tb_last_error() (bins/nnue_train/src/trainer_common.rs:313
 *    maps such errors to io::Error::other).
 *  - one caller thread per handle (the reference's trainers are Send, not Sync).
 *  - pageable host input arrays are copied into the library's own pinned ring before a
 *    call returns, so the caller may reuse them immediately (InputUploadRing,
 *    bins/nnue_train/src/trainer_common.rs:1041-1097).  Page-locked arrays (tb_host_alloc,
 *    cudaHostAlloc) are read by the copy engine directly: keep batch k untouched until
 *    tb_train_step(k+1) returns, the recycling rule of the reference's training loop
 *    (crates/nnue-train/src/trainer.rs:925-994).
 *  - tb_train_step reports the loss sum of the PREVIOUS step; the first call reports 0.0
 *    (AsyncLossRing, bins/nnue_train/src/trainer_common.rs:909-976).
 */
#ifndef TATARA_B200_H
#define TATARA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB_OK 0
#define TB_ERR_INVALID_ARGUMENT (-1)
#define TB_ERR_CUDA (-2)
#define TB_ERR_OUT_OF_MEMORY (-3)
#define TB_ERR_UNSUPPORTED (-4)
#define TB_ERR_NCCL (-5)
#define TB_ERR_NO_DEVICE (-6)
#define TB_ERR_TIMEOUT (-7) /* a data-parallel step did not finish within the deadline: a peer is gone; the handle is poisoned */

enum { TB_ARCH_LAYERSTACK = 0, TB_ARCH_SIMPLE = 1 };
/* SimpleActivation (bins/nnue_train/src/trainer_simple.rs): Pairwise is the FT-output pairwise product of the LayerStack
 * net (the L1 input is then ft_out wide instead of 2 * ft_out); L1 and L2 are CReLU then */
enum { TB_ACT_CRELU = 0, TB_ACT_SCRELU = 1, TB_ACT_PAIRWISE = 2 };
/* crates/nnue-train/src/optimizer.rs:32-37 OptimizerKind */
enum { TB_OPT_RANGER = 0, TB_OPT_RADAM = 1, TB_OPT_ADAMW = 2 };
/* bins/nnue_train/src/cli.rs:623-638 precision flags; --all-optim sets all four.  Accepted for LayerStack with l1_out of 8,
 * 16 or 32 (TB_ERR_UNSUPPORTED otherwise).  TF32: the L1 forward product runs on the tensor cores with TF32 operands (the
 * reference: cuBLAS TF32 tensor-op mode); FT_FP16: fp16 forward table; FT_FP16_OUT (needs FT_FP16): fp16 pre-activations and
 * fp16 FT gradient rows scaled by 2^14 * batch and clamped to +-65504; FP16_OPT_STATE: fp16 moments of the FT table, scaled
 * by 2^28 / 2^40 (bins/nnue_train/src/arch.rs:72-93).  Uploads and downloads stay fp32. */
enum { TB_PREC_TF32 = 1, TB_PREC_FT_FP16 = 2, TB_PREC_FT_FP16_OUT = 4, TB_PREC_FP16_OPT_STATE = 8 };
enum { TB_LOSS_SIGMOID = 0, TB_LOSS_WRM = 1 };

typedef struct tb_trainer tb_trainer;

/*
 * Construction parameters.  Replaces the argument lists of GpuTrainer::new
 * (bins/nnue_train/src/trainer_layerstack.rs:781-796) and SimpleGpuTrainer::new
 * (bins/nnue_train/src/trainer_simple.rs:392-402).  The feature set is passed by its
 * dimensions (crates/shogi-features/src/feature_set.rs:1031-1038) instead of by name.
 */
#define TB_DP_NCCL 0
#define TB_DP_PEER_COPY 1
#define TB_DP_PEER_KERNEL 2

typedef struct tb_config {
    int32_t struct_size;    /* sizeof(tb_config) of the caller */
    int32_t device;         /* CUDA device ordinal */
    int32_t arch;           /* TB_ARCH_* */
    int32_t batch_capacity; /* largest n_pos a step may carry; multiple of 16 */
    int32_t ft_in;          /* N: real feature rows */
    int32_t piece_inputs;   /* pi: rows per king bucket (N = king_buckets * pi) */
    int32_t ft_factorize;   /* 1: pi virtual rows are trained on top (train rows = N + pi) */
    int32_t max_active;     /* A: slots per position and perspective */
    int32_t ft_out;         /* F: multiple of 128 (bins/nnue_train/src/arch.rs:13-19) */
    int32_t l1_out;         /* LayerStack: includes the skip output; Simple: hidden 1 */
    int32_t l2_out;
    int32_t num_buckets;    /* LayerStack: 2..9; ignored for Simple */
    int32_t activation;     /* Simple: TB_ACT_* (CReLU, SCReLU, Pairwise); LayerStack is always pairwise CReLU */
    int32_t optimizer;      /* TB_OPT_* */
    int32_t precision;      /* bit mask of TB_PREC_* */
    float wd_ft, wd_dense, wd_bias;                /* OptimGroupConfig, trainer_layerstack.rs:640-705 */
    float lr_mult_ft, lr_mult_dense, lr_mult_bias; /* Simple uses wd_ft / lr_mult_ft for every group */
    int32_t world_size;     /* data-parallel ranks (1 = single GPU, NCCL not loaded) */
    int32_t rank;
    uint8_t nccl_unique_id[128]; /* from tb_nccl_unique_id() on rank 0, same bytes on every rank */
    int32_t nccl_ctas;      /* > 0: this handle's communicator is created by ncclCommInitRankConfig with minCTAs = maxCTAs =
                               this value (a fixed channel count); 0: ncclCommInitRank, NCCL chooses.  Algorithm, protocol and
                               NVLS have no per-communicator setting in NCCL: they are the application's NCCL_ALGO, NCCL_PROTO
                               and NCCL_NVLS_ENABLE, which this library neither sets nor changes. */
    int32_t dp_exchange;    /* TB_DP_NCCL (0): the gradient parts are summed by ncclAllReduce.  TB_DP_PEER_COPY (1): ranks of
                               one node, one process each: reduce-scatter and all-gather by the copy engines over peer
                               mappings (CUDA IPC) with stream memory operations as signals and a small summing kernel in
                               rank order; NCCL then only carries the start-up handshake and batches off the fast path.
                               TB_DP_PEER_KERNEL (2): the same signals, the data moved by one kernel per part that reads every
                               rank's shard over the peer mappings, sums in rank order and stores the sum to every rank */
} tb_config;

/* nnue_train::trainer::LossKind, crates/nnue-train/src/trainer.rs:75-95 */
typedef struct tb_loss {
    int32_t kind; /* TB_LOSS_* */
    float scale;  /* sigmoid: 1 / scale_param */
    float nnue2score, in_scaling, in_offset, target_offset, target_scaling;
    float pow_exp, qp_asymmetry, weight_boost_w1, weight_boost_w2;
} tb_loss;

/* BatchData, bins/nnue_train/src/trainer_common.rs:142-151.  All pointers are HOST memory. */
typedef struct tb_batch {
    int32_t n_pos;               /* multiple of 16, <= batch_capacity */
    const int32_t* stm_indices;  /* [n_pos, A]; slots >= nnz are ignored; out-of-range values are skipped */
    const int32_t* nstm_indices; /* [n_pos, A] */
    const int32_t* nnz;          /* [n_pos], shared by both perspectives */
    const int32_t* bucket_idx;   /* [n_pos] LayerStack; NULL for Simple */
    const float* score;          /* [n_pos] raw centipawns */
    const float* wdl;            /* [n_pos] 0 / 0.5 / 1 */
    float per_pos_norm;          /* 0 selects the reference's 1 / (n_pos * world_size) */
} tb_batch;

/* ---- life cycle ------------------------------------------------------------------ */
int tb_create(const tb_config* cfg, tb_trainer** out);
/* synchronises both streams before freeing (Drop, trainer_layerstack.rs:335-347) */
void tb_destroy(tb_trainer* t);
/* text of the last error on this handle; with NULL, of the last failed tb_create on this thread */
const char* tb_last_error(const tb_trainer* t);

/* ---- parameter groups -------------------------------------------------------------
 * Names and order follow raw_ckpt_group_sources / uniform_optim_group_layout
 * (trainer_layerstack.rs:740-762): ft_w, ft_b, l1_w, l1_b, l1_shared_weight,
 * l1_shared_bias, l2_w, l2_b, l3_w, l3_b; Simple: ft_w, ft_b, l1_w ([2 * ft_out, l1]; Pairwise [ft_out, l1]), l1_b, l2_w,
 * l2_b, l3_w, l3_b.  Initial weights always come from the host (init.rs or a checkpoint). */
int tb_num_groups(const tb_trainer* t);
const char* tb_group_name(const tb_trainer* t, int group);
int64_t tb_group_len(const tb_trainer* t, const char* name);
/* NULL pointers are skipped.  Re-derives the forward table (factorizer fold) like
 * sync_ft_forward_weights.  Moments are true f32 values (MomentBuf::to_host_f32,
 * trainer_common.rs:89-126). */
int tb_upload_group(tb_trainer* t, const char* name, const float* w, const float* m, const float* v,
                    const float* slow, int64_t len);
int tb_download_group(tb_trainer* t, const char* name, float* w, float* m, float* v, float* slow, int64_t len);
int tb_get_step_count(const tb_trainer* t, uint64_t* step_count);
int tb_set_step_count(tb_trainer* t, uint64_t step_count);

/* ---- the step (trait TrainerBackend, crates/nnue-train/src/trainer.rs:273-374) ------ */
/* train_step -> GpuTrainer::step (trainer_layerstack.rs:1885) / SimpleGpuTrainer::step
 * (trainer_simple.rs:742).  n_pos == 0 returns loss 0 without work. */
int tb_train_step(tb_trainer* t, const tb_batch* batch, float lr, float wdl_lambda, const tb_loss* loss,
                  double* loss_prev);
/* train_step fed with PackedSfenValue records instead of extracted indices: `psv` is n_pos 40-byte records in HOST
 * memory (crates/shogi-format/src/packed_sfen.rs:251-271); 40 bytes per position cross the bus and the work of the
 * reference's dataloader workers (decode, feature extraction of both perspectives, kingrank9 bucket, score and wdl:
 * crates/nnue-train/src/dataloader.rs:444-500, 1303-1407) runs on the device on the copy stream, overlapped with the
 * previous step.  feature_set as in tb_psv_extract; it must be the set the trainer was created for.  The step is
 * bit-identical to tb_train_step on the batch tb_psv_extract returns for the same records.  per_pos_norm is the
 * reference's 1 / (n_pos * world_size). */
int tb_train_step_psv(tb_trainer* t, int feature_set, const uint8_t* psv, int n_pos, float lr, float wdl_lambda,
                      const tb_loss* loss, double* loss_prev);
/* flush_pending_loss: the lagged loss of the last step, then re-arms the ring */
int tb_flush_pending_loss(tb_trainer* t, double* loss);
/* validate_step -> GpuTrainer::validate (trainer_layerstack.rs:1963): forward + loss only, no state
 * change; net_output receives n_pos values */
int tb_validate_step(tb_trainer* t, const tb_batch* batch, float wdl_lambda, const tb_loss* loss,
                     double* sum_sq_err, float* net_output);
/* read_fp16_clamp_count (trainer.rs:368-373): fp16 FT gradient elements that hit the clamp, and elements written, since
 * the handle was created; both 0 without TB_PREC_FT_FP16_OUT */
int tb_read_fp16_clamp_count(tb_trainer* t, uint64_t* clamps, uint64_t* elems);

/* ---- device-resident batches -------------------------------------------------------
 * A batch may be uploaded once into one of TB_NUM_SLOTS device slots and stepped on
 * repeatedly (the reference's native-bench runs a fixed in-memory batch,
 * bins/nnue_train/src/native_bench.rs:550-576). */
#define TB_NUM_SLOTS 4 /* slots 0..2 are the caller's; the last one is the library's scratch batch */
int tb_stage_batch(tb_trainer* t, int slot, const tb_batch* batch);
int tb_train_step_staged(tb_trainer* t, int slot, float lr, float wdl_lambda, const tb_loss* loss,
                         double* loss_prev);

/* ---- diagnostics used by the parity tests ------------------------------------------- */
/* forward + backward (+ gradient all-reduce when world_size > 1) without the optimizer; returns this
 * step's own loss sum, synchronously */
int tb_forward_backward(tb_trainer* t, const tb_batch* batch, float wdl_lambda, const tb_loss* loss,
                        double* loss_now);
/* runs the optimizer on the gradients currently held (completes a tb_forward_backward) */
int tb_apply_optimizer(tb_trainer* t, float lr);
/* gradient of a group after tb_forward_backward */
int tb_download_grad(tb_trainer* t, const char* name, float* grad, int64_t len);
/* an intermediate of the last step in the caller's position order: "ft_stm", "ft_nstm", "combined",
 * "l1_total", "net_output", "dy", "dl1_total", "dft_stm", "dft_nstm", "comb" */
int tb_read_buffer(tb_trainer* t, const char* name, float* out, int64_t len);

/* ---- timing --------------------------------------------------------------------------
 * CUDA events on the library's compute stream.  With profiling on, every kernel phase of a step is
 * bracketed by events; tb_profile_read returns the accumulated milliseconds and launch counts. */
int tb_timer_start(tb_trainer* t);
int tb_timer_stop(tb_trainer* t, float* elapsed_ms);
int tb_profile_enable(tb_trainer* t, int on);
int tb_profile_num_phases(const tb_trainer* t);
int tb_profile_read(tb_trainer* t, int phase, const char** name, double* total_ms, int64_t* launches);
int tb_profile_reset(tb_trainer* t);
/* kernels launched by this handle since creation */
int64_t tb_launch_count(const tb_trainer* t);
int tb_synchronize(tb_trainer* t);

/* ---- FT kernels alone (the reference's per-kernel microbenchmark shapes) ---------------
 * Device-resident single-perspective runs of the three FT kernels on caller-provided HOST data.
 * forward: out[b, :] = sum of table rows (native_kernels.cu:162 sparse_ft_forward);
 * backward: grad[f, :] = sum of dft rows whose position lists f (native_kernels.cu:1630-1840);
 * adam: one fused AdamW + clamp pass (native_kernels.cu:1291 radam_step with scalars (1, 1)).
 * `iters` launches are timed with events; results are copied back when the output pointer is not NULL. */
int tb_ft_forward_bench(int device, const float* table, const int32_t* indices, const int32_t* nnz,
                        int batch, int ft_out, int ft_in, int max_active, int iters, float* out, float* ms_per_iter);
int tb_ft_backward_bench(int device, const float* dft, const int32_t* indices, const int32_t* nnz,
                         int batch, int ft_out, int ft_in, int max_active, int iters, float* grad, float* ms_per_iter);
int tb_adam_clamp_bench(int device, float* w, float* m, float* v, const float* grad, int64_t n, float lr,
                        float decay, float min_w, float max_w, int iters, float* ms_per_iter);

/* The three FT kernels on DEVICE-resident data, one perspective (the reference's microbenchmark protocol:
 * a fixed in-memory batch, warm-up, timed launches, bins/nnue_train/src/native_bench.rs:550-576,
 * docs/native-cuda-benchmark.md:11-33).  Only the index lists come from the host; table, incoming gradient rows and
 * moments are filled on the device.  Every launch group is timed with its own pair of CUDA events; with flush_l2 a
 * 256 MB buffer is written before each one.  fwd / bwd / adam: the generic kernels (L2 gather; global inverse index +
 * per-row sums; AdamW with the +-32767/127 clamp).  With rows_per_slice > 0 and king-sliced lists (every row of a
 * position inside one slice of rows_per_slice table rows) the slice-resident kernels of the training step are timed
 * too, sorts and plans included; otherwise those two fields are negative. */
typedef struct tb_ft_microbench_result {
    float fwd_ms, bwd_ms, adam_ms;
    float fwd_slice_ms, bwd_slice_ms;
    int32_t iters;
} tb_ft_microbench_result;
int tb_ft_microbench(int device, const int32_t* indices, const int32_t* nnz, int batch, int ft_out, int ft_in,
                     int rows_per_slice, int max_active, int iters, int flush_l2, tb_ft_microbench_result* out);

/* ---- FT weight gradient without any allocation -------------------------------------------
 * No counterpart in the reference (its trainers allocate their workspace in the constructor).
 * For hosts that must not allocate device memory once they run — a framework whose allocator owns the
 * whole GPU, a process with a fixed memory plan — this variant of the FT backward keeps the working
 * memory of the inverse index and of the long-list partial sums in a static device array inside the
 * library (about 21.5 MB per GPU, held until exit) and calls no cudaMalloc / cudaFree.  ALL pointers are DEVICE memory owned by the caller;
 * the work is enqueued on `stream` (a cudaStream_t, NULL = default stream) and not synchronised.
 * Limits: ft_in <= TB_STATIC_SCRATCH_MAX_FT_IN and batch * max_active <= TB_STATIC_SCRATCH_MAX_PAIRS;
 * beyond them the call fails and writes the reason to err (may be NULL).  Calls share the one array:
 * never let two of them overlap on a GPU.  The first call on a device resolves the array's address;
 * issue it before any stream capture.  d_dft and d_grad must be 16-byte aligned (rows move as 128-bit
 * vectors).  Same kernels and same summation order as tb_ft_backward_bench (lists of more than 4096 entries are
 * summed in parts of 4096), so the two agree bit for bit. */
#define TB_STATIC_SCRATCH_MAX_FT_IN 131072
#define TB_STATIC_SCRATCH_MAX_PAIRS 655360
int tb_ft_backward_static_scratch(const float* d_dft, const int32_t* d_indices, const int32_t* d_nnz, int batch,
                                  int ft_out, int ft_in, int max_active, float* d_grad, void* stream, char* err,
                                  size_t err_len);

/* ---- inputs: PackedSfenValue records -> step inputs, on the device ---------------------
 * Decodes 40-byte records (crates/shogi-format/src/packed_sfen.rs:387-448) and extracts the active
 * feature indices of both perspectives (crates/shogi-features/src/feature_set.rs:655-808), the
 * kingrank9 bucket (crates/shogi-features/src/kingrank9.rs:11-24), score and wdl
 * (crates/nnue-train/src/dataloader.rs:444-500).  feature_set: 0 halfkp, 4 halfka-hm-merged.
 * All pointers are HOST memory; bucket may be NULL. */
int tb_psv_extract(int device, int feature_set, const uint8_t* psv, int64_t n_records, int32_t* stm_indices,
                   int32_t* nstm_indices, int32_t* nnz, int32_t* bucket, float* score, float* wdl);
/* seeded synthetic PackedSfenValue records (host): full 40-piece sets, see the generator's comment */
int tb_psv_synthesize(uint64_t seed, int64_t n_records, uint8_t* psv_out);
/* encodes one position (host); arrays as in the decoder's board: piece type 0..14, colour 0/1 */
int tb_psv_encode(const uint8_t* board_pt, const uint8_t* board_color, const uint8_t* hand_black7,
                  const uint8_t* hand_white7, int side_to_move, int black_king_sq, int white_king_sq,
                  int score, int ply, int result, uint8_t* psv40_out);

/* ---- weight initialisation (host) --------------------------------------------------------
 * The reference's deterministic sampler (crates/nnue-train/src/init.rs:111-210), for callers that have
 * no Rust host to draw the initial weights.  dist: 0 zeroed, 1 uniform.  scale_kind: 0 absolute half
 * width, 1 sqrt(scale_value / fan_in). */
int tb_init_sample(float* out, int64_t n, int64_t num_buckets, int64_t fan_in, int dist, int scale_kind,
                   float scale_value, int per_bucket_repeat, uint64_t seed);

/* page-locked host memory for step inputs (pinned_host_alloc of the reference's runtime,
 * crates/cuda-native-runtime/src/runtime.rs:701-769) */
int tb_host_alloc(void** out, size_t bytes);
int tb_host_free(void* p);

/* ---- data parallel ---------------------------------------------------------------------- */
/* rank 0 creates the id, every rank passes the same bytes in tb_config.nccl_unique_id */
int tb_nccl_unique_id(uint8_t out[128]);

int tb_device_count(void);
const char* tb_version(void);

#ifdef __cplusplus
}
#endif
#endif
