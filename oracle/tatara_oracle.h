/*
 * CPU oracle for the NNUE training step — TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement of tatara's per-kernel CPU reference functions
 * (the crates/gpu-kernels sources), its PackedSfenValue decoder and feature
 * extractors (crates/shogi-format, crates/shogi-features), its weight
 * initialiser and optimizer scalars (crates/nnue-train/src/{init,optimizer}.rs),
 * composed into whole-step functions that follow the launch order of
 * bins/nnue_train/src/trainer_{layerstack,simple}.rs.
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may link
 * or call this library.  The CUDA library never does.
 *
 * Parity status: every per-kernel function is pinned by the literal vectors of
 * the reference's own unit tests (tests/test_oracle_golden.py).  The composed
 * whole-step functions have no runnable reference counterpart (the reference
 * pins them only with GPU-vs-GPU tests that need Rust and a GPU): at that level
 * parity is unpinned.
 */
#ifndef TATARA_ORACLE_H
#define TATARA_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- sparse feature transformer ------------------------------------------------ */
void ora_sparse_ft_forward(const float* weight, const int32_t* indices, const int32_t* nnz_arr,
                           float* out, size_t batch, size_t rows, size_t cols, size_t max_active);
void ora_sparse_ft_backward(const float* grad_out, const int32_t* indices, float* grad_weight,
                            size_t batch, size_t rows, size_t cols, size_t nnz);
void ora_ft_fold_virtual(const float* w, float* comb, size_t ft_in, size_t ft_out, size_t piece_inputs);
void ora_ft_reduce_virtual_grad(float* grad, size_t ft_in, size_t ft_out, size_t piece_inputs);

/* ---- LayerStack pieces --------------------------------------------------------- */
void ora_ft_post_perspective_fwd(const float* stm, const float* nstm, const float* bias,
                                 float* combined, size_t batch, size_t ft_dim, float scale);
void ora_ft_post_perspective_grad(const float* d_combined, const float* ft_out, const float* bias,
                                  float* grad_ft_out, float* grad_bias, size_t batch, size_t ft_dim,
                                  size_t d_combined_offset, size_t d_combined_stride, float scale);
void ora_dense_mm_fwd(const float* x, const float* w, const float* bias, float* y,
                      size_t batch, size_t in_dim, size_t out_dim);
void ora_dense_mm_bwd_input(const float* dy, const float* w, float* dx,
                            size_t batch, size_t in_dim, size_t out_dim);
void ora_dense_mm_bwd_weight(const float* x, const float* dy, float* grad_w,
                             size_t batch, size_t in_dim, size_t out_dim);
void ora_bias_grad(const float* dy, float* grad_bias, size_t batch, size_t out_dim);
void ora_dense_mm_fwd_bucket(const float* x, const float* w, const float* bias, const int32_t* bucket_idx,
                             float* y, size_t batch, size_t in_dim, size_t out_dim, size_t num_buckets);
void ora_dense_mm_bwd_input_bucket(const float* dy, const float* w, const int32_t* bucket_idx, float* dx,
                                   size_t batch, size_t in_dim, size_t out_dim, size_t num_buckets);
void ora_dense_mm_bwd_weight_bucket(const float* x, const float* dy, const int32_t* bucket_idx,
                                    float* grad_w, size_t batch, size_t in_dim, size_t out_dim,
                                    size_t num_buckets);
void ora_bias_grad_bucket(const float* dy, const int32_t* bucket_idx, float* grad_bias,
                          size_t batch, size_t out_dim, size_t num_buckets);
void ora_crelu_fwd(const float* x, float* y, size_t n);
void ora_crelu_grad(const float* x, const float* dy, float* dx, size_t n);
void ora_screlu_fwd(const float* x, float* y, size_t n);
void ora_screlu_grad(const float* x, const float* dy, float* dx, size_t n);
void ora_abs_pow2_scale_fwd(const float* x, float* y, float scale, size_t n);
void ora_abs_pow2_scale_grad(const float* x, const float* dy, float* dx, float scale, size_t n);
void ora_concat_l1sqr_main_fwd(const float* a, const float* b, float* out, size_t batch, size_t a_dim, size_t b_dim);
void ora_concat_l1sqr_main_grad(const float* dout, float* da, float* db, size_t batch, size_t dim);
void ora_slice_extract_2d(const float* src, float* dst, size_t batch, size_t src_stride, size_t src_offset, size_t out_dim);
void ora_slice_scatter_2d(const float* src, float* dst, size_t batch, size_t in_dim, size_t dst_stride, size_t dst_offset);
void ora_elementwise_add(const float* a, const float* b, float* c, size_t n);

/* ---- losses -------------------------------------------------------------------- */
void ora_loss_wdl(const float* out, const float* score, const float* wdl, const float* per_pos_norm,
                  float* dl_dout, double* loss_acc, float lambda, float scale, size_t n);
void ora_loss_wrm(const float* out, const float* score, const float* wdl, const float* per_pos_norm,
                  float* dl_dout, double* loss_acc, float lambda, float nnue2score, float in_scaling,
                  float in_offset, float target_offset, float target_scaling, float pow_exp,
                  float qp_asymmetry, float weight_boost_w1, float weight_boost_w2, int extended, size_t n);

/* ---- optimizer ----------------------------------------------------------------- */
void ora_radam_compute_step_size_denom(uint64_t step, float beta1, float beta2, float n_sma_threshold,
                                       float* step_size, int32_t* denom);
void ora_radam_step(float* weights, float* m, float* v, float* grad, float lr, float step_size,
                    int32_t denom, float decay, float beta1, float beta2, float eps,
                    float min_w, float max_w, size_t n);
void ora_ranger_lookahead_lerp(float* weights, float* slow, float alpha, size_t n);
/* kind: 0 = ranger, 1 = radam, 2 = adamw */
void ora_optimizer_scalars(int kind, uint64_t step, float beta2, float n_sma_threshold,
                           float* step_size, int32_t* denom, float* beta1);

/* ---- weight init ---------------------------------------------------------------- */
/* dist: 0 zeroed, 1 uniform.  scale_kind: 0 Abs(value), 1 FanIn{gain=value}. */
void ora_init_sample(float* out, size_t n, size_t num_buckets, size_t fan_in, int dist,
                     int scale_kind, float scale_value, int per_bucket_repeat, uint64_t seed);

/* ---- PackedSfenValue / features -------------------------------------------------- */
typedef struct {
    uint8_t board_pt[81];    /* PieceType discriminant, 0 = none */
    uint8_t board_color[81]; /* 0 black, 1 white */
    uint8_t hand[2][7];      /* [color][pawn,lance,knight,silver,gold,bishop,rook] */
    uint8_t side_to_move;
    uint8_t black_king_sq, white_king_sq;
    int16_t score;
    int8_t result;
    uint16_t ply;
} ora_board;

void ora_psv_decode(const uint8_t* psv40, ora_board* out);
/* inverse of the decoder, and the benchmark's seeded synthetic record generator (see the .c file for its draw order) */
int ora_psv_encode(const ora_board* b, uint8_t* psv40_out);
int ora_psv_synthesize(uint64_t seed, size_t n_records, uint8_t* out);
/* feature_set: 0 halfkp, 1 halfka-split, 2 halfka-merged, 3 halfka-hm-split, 4 halfka-hm-merged */
int ora_feature_dims(int feature_set, int* king_buckets, int* piece_inputs, int* ft_in, int* max_active);
int ora_extract_active_features(int feature_set, const ora_board* board, int32_t* stm_out,
                                int32_t* nstm_out, int cap);
int ora_kingrank9_bucket(const ora_board* board);
/* whole batch: PSV records -> the trainer's step inputs (dataloader Batch::push_decoded). */
int ora_psv_to_batch(int feature_set, const uint8_t* psv, size_t n_records, int32_t* stm_idx,
                     int32_t* nstm_idx, int32_t* nnz, int32_t* bucket, float* score, float* wdl);
/* loader-digest message bytes for one position (bins/nnue_train/src/loader_digest.rs). */
size_t ora_loader_digest_bytes(const int32_t* stm, const int32_t* nstm, int32_t nnz, float score,
                               float wdl, uint8_t* out);

/* ---- whole-step trainers --------------------------------------------------------- */
typedef struct {
    int arch;         /* 0 = LayerStack, 1 = Simple */
    int ft_in;        /* N */
    int piece_inputs; /* pi */
    int factorize;    /* 1: train rows = N + pi */
    int max_active;   /* A */
    int ft_out;       /* F */
    int l1, l2;
    int num_buckets;  /* LayerStack only */
    int activation;   /* Simple: 0 crelu, 1 screlu */
    int optimizer;    /* 0 ranger, 1 radam, 2 adamw */
    float wd_ft, wd_dense, wd_bias;
    float lr_mult_ft, lr_mult_dense, lr_mult_bias;
} ora_config;

typedef struct {
    int kind; /* 0 sigmoid {scale}, 1 wrm */
    float scale;
    float nnue2score, in_scaling, in_offset, target_offset, target_scaling;
    float pow_exp, qp_asymmetry, weight_boost_w1, weight_boost_w2;
} ora_loss;

typedef struct ora_trainer ora_trainer;

ora_trainer* ora_trainer_create(const ora_config* cfg, int batch_capacity);
void ora_trainer_destroy(ora_trainer* t);
int ora_trainer_num_groups(const ora_trainer* t);
const char* ora_trainer_group_name(const ora_trainer* t, int g);
size_t ora_trainer_group_len(const ora_trainer* t, int g);
/* which: 0 w, 1 m, 2 v, 3 slow, 4 grad (grad holds the last step's gradient) */
float* ora_trainer_group_ptr(ora_trainer* t, int g, int which);
/* default initialisation of the reference (init.rs default_uniform for the arch). */
void ora_trainer_init_default(ora_trainer* t);
uint64_t ora_trainer_step_count(const ora_trainer* t);
void ora_trainer_set_step_count(ora_trainer* t, uint64_t s);
void ora_trainer_set_threads(ora_trainer* t, int n_threads);
/* named workspace buffer after a step (e.g. "ft_stm", "combined", "l1_total", "net_output", "dy",
 * "dft_stm", "dft_nstm"); returns NULL when unknown. */
const float* ora_trainer_buffer(const ora_trainer* t, const char* name, size_t* len);
/* One training step.  per_pos_norm is the scalar 1/n_pos (or 1/(world*n_pos) for data parallel).
 * do_optimizer = 0 stops after backward (gradients stay in the grad buffers).
 * Returns the un-normalised loss sum of THIS step. */
double ora_trainer_step(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                        const int32_t* bucket_idx, const float* score, const float* wdl, int n_pos,
                        float per_pos_norm, float lr, float wdl_lambda, const ora_loss* loss,
                        int do_optimizer);
/* forward + loss only; net_output[n_pos] filled. */
double ora_trainer_validate(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                            const int32_t* bucket_idx, const float* score, const float* wdl, int n_pos,
                            float wdl_lambda, const ora_loss* loss, float* net_output);
/* adds every gradient buffer of `src` into `dst` (data-parallel emulation: rank order = call order). */
void ora_trainer_accumulate_grads(ora_trainer* dst, const ora_trainer* src);
/* runs only the optimizer part on the gradients currently held. */
void ora_trainer_apply_optimizer(ora_trainer* t, float lr);
/* reduced precision of the LayerStack trainer: bit 1 tf32, 2 ft_fp16, 4 ft_fp16_out, 8 fp16_opt_state */
void ora_trainer_set_precision(ora_trainer* t, int flags);
void ora_trainer_clamp_count(const ora_trainer* t, uint64_t* clamps, uint64_t* elems);
float ora_round_half(float x);
float ora_tf32(float x);
void ora_radam_step_f16state(float* weights, float* m, float* v, float* grad, float lr, float step_size, int32_t denom,
                             float decay, float beta1, float beta2, float eps, float min_w, float max_w, float m_scale,
                             float v_scale, size_t n);

#ifdef __cplusplus
}
#endif
#endif
