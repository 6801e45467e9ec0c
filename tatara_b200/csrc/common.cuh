// Shared declarations of the sm_100a NNUE training-step library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define TB_MAX_BUCKETS 9  // kMaxSupportedNumBuckets of the reference (native_kernels.cu:9)
#define TB_MAX_L1 32
#define TB_MAX_L2 64
#define TB_TILE_M 32      // positions per dense tile; a tile never mixes LayerStack buckets
#define TB_UNIT_TILES 8   // tiles per work unit (consecutive tiles of one bucket)

// One tile of positions for the bucket-grouped dense kernels: positions order[start .. start+count).
// bucket == num_buckets marks positions whose bucket id is out of range (their per-bucket layers
// output zero, dense_mm_bucket.rs:45-73).
struct TileDesc {
    int start;
    int count;
    int bucket;
    int pad;
};

struct LossParams {
    int kind;  // 0 sigmoid, 1 wrm
    float scale;
    float nnue2score, in_scaling, in_offset, target_offset, target_scaling;
    float lambda;
    float norm;  // per-position gradient normaliser
    // extended WRM (LossKind::wrm_extended, crates/nnue-train/src/trainer.rs:127-137): error power, asymmetry, per-position
    // weights normalised by their sum over the batch (*weight_sum, on the device, filled by launch_wrm_weight_sum)
    int extended = 0;
    float pow_exp = 2.0f, qp_asymmetry = 0.0f, w1 = 0.0f, w2 = 0.5f;
    float n_pos = 0.0f;
    const double* weight_sum = nullptr;
};

struct OptScalars {
    float lr, step_size, decay, beta1, beta2, eps, min_w, max_w, alpha;
    int denom;
    int lerp;  // apply the Ranger look-ahead interpolation after the update
    // Factor the stored gradient is multiplied by on load (1 unless the FT weight gradient was summed from loss-scaled
    // fp16 rows: then the inverse of that scale).  Applies to the real FT rows only.
    float grad_scale = 1.0f;
};
// fp16 optimizer state of the FT table: m is stored as m * 2^28, v as v * 2^40, clamped to the fp16 range
// (bins/nnue_train/src/arch.rs:95-117 FT_OPT_M_SCALE / FT_OPT_V_SCALE; radam_step_f16state, native_kernels.cu:1127-1181)
#define TB_FT_OPT_M_SCALE 268435456.0f
#define TB_FT_OPT_V_SCALE 1099511627776.0f

// One small parameter group for the batched optimizer kernel.
struct SmallGroup {
    float *w, *m, *v, *slow;
    const float* grad;
    int n;
    float lr, decay, min_w, max_w;
};
#define TB_MAX_SMALL_GROUPS 12
// passed to the kernel by value (kernel parameter space), so no per-step upload is needed
struct SmallGroups {
    SmallGroup g[TB_MAX_SMALL_GROUPS];
    int n;
};

static __device__ __forceinline__ float crelu01(float x) { return x < 0.0f ? 0.0f : (x > 1.0f ? 1.0f : x); }

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- launchers (each returns the number of kernels it launched) --------------------------------

// ft_kernels.cu
// mode: 0 raw gather-sum, 1 LayerStack pairwise (+bias, CReLU, product, scale), 2 Simple CReLU, 3 Simple SCReLU
// items: the (position, perspective) processing order from launch_step_sorts, or NULL for natural order
int launch_ft_forward(cudaStream_t s, int mode, const void* table, const int* idx_stm, const int* idx_nstm,
                      const int* nnz, const float* bias, void* pre_stm, void* pre_nstm, float* combined,
                      const int* items, int B, int F, int N, int A, float scale, int n_persp, int table_half = 0,
                      int out_half = 0);
// slice-resident forward: every item's rows come from a 32-column strip of its king-bucket slice held in shared
// memory.  Needs items / item_seg from launch_step_sorts with the same rows_per_slice; work: scratch of
// ft_forward_slice_work_ints(n_items, slices + 1, A) ints.
bool ft_forward_slice_supported(int F, int N, int A, int rows_per_slice);
size_t ft_forward_slice_work_ints(int n_items, int n_keys, int A);
// table_half: fp16 table rows (64-column strips); out_half: fp16 pre-activations (needs table_half).  Returns -1 for a
// combination that is not built (fp16 with the Simple activations).
int launch_ft_forward_slice(cudaStream_t s, int mode, const void* table, const int* idx_stm, const int* idx_nstm,
                            const int* nnz, const float* bias, void* pre_stm, void* pre_nstm, float* combined,
                            const int* items, const int* item_seg, int* work, int B, int F, int N, int A,
                            int rows_per_slice, float scale, int n_persp, int table_half = 0, int out_half = 0);
// scratch of the inverse index, in ints: histogram [2N], a counter, a queue of long lists [2N], scan block sums
static inline size_t inverse_index_counts_len(int N) { return 4 * (size_t)N + 1 + 2 * ((size_t)N / 2048 + 2); }
// counts: [inverse_index_counts_len(N)], offsets: [2][N+1], cursor: [2][N], lists: [4][B*A] (lists + sort scratch)
// run_if (here and below): NULL, or a device flag; the launched kernels return at once while it is 0
int launch_inverse_index(cudaStream_t s, const int* run_if, const int* idx_stm, const int* idx_nstm, const int* nnz, int B, int A,
                         int N, int n_persp, int* counts, int* offsets, int* cursor, int* lists);
// long lists are cut into parts summed by separate blocks; plan: [2 + 2 * max_work + 3 * N] ints,
// partial: [max_work][F] floats with max_work = ft_backward_max_work(B, A, n_persp)
int ft_backward_max_work(int B, int A, int n_persp);
// dft_half: the incoming gradient rows are fp16; the sums keep the rows' loss scale
int launch_ft_backward_split(cudaStream_t s, const int* run_if, const void* dft_stm, const void* dft_nstm, const int* offsets,
                             const int* lists, int B, int A, int N, int F, int n_persp, int* plan, float* partial,
                             float* grad, int dft_half = 0);
// slice-resident weight gradient (ft_slice_bwd.cu).  Needs the slice-resident forward of the same step (its row codes
// in fwd_work) and items / item_seg of the same rows_per_slice; bwd_work: ft_backward_slice_ints(...) ints.  The kernels
// do nothing when the batch has a row outside its item's slice: *ft_slice_outside_flag(...) is then 1 and the generic
// kernels, launched with it as run_if, do the work instead.
bool ft_backward_slice_supported(int F, int N, int A, int rows_per_slice);
size_t ft_backward_slice_ints(int n_items, int A, int rows_per_slice);
// floats of the partial slabs launch_ft_backward_slice needs (slices of many chunks are shared by several blocks)
size_t ft_backward_slice_slab_floats(int n_items, int A, int rows_per_slice, int F);
const int* ft_slice_outside_flag(int* fwd_work, int n_items, int N, int rows_per_slice);
int launch_inverse_slice(cudaStream_t s, const int* item_seg, int* fwd_work, int* bwd_work, int B, int A, int N,
                         int rows_per_slice, int n_persp);
// the rows of slices [slice_begin, slice_begin + slice_count)
int launch_ft_backward_slice(cudaStream_t s, const void* dft_stm, const void* dft_nstm, int* fwd_work, int* bwd_work, int B,
                             int A, int N, int F, int rows_per_slice, int n_persp, int slice_begin, int slice_count, float* grad,
                             float* slabs, int dft_half = 0);
int sort_max_units(int max_tiles);
// The two sorts of a step: positions by bucket -> order, bucket segments seg_start [nb + 2], tiles (room for max_tiles
// tiles followed by the work units; n_tiles is {tile count, unit count}); items (position, perspective) of both
// perspectives by the table slice of their features -> items, item_seg [slices + 2].  hist: scratch of
// (nb + 1) * ceil(B / 1024) + (slices + 1) * ceil(n_persp * B / 1024) ints
int launch_step_sorts(cudaStream_t s, const int* bucket /*may be NULL*/, int B, int nb, int* order, TileDesc* tiles, int* n_tiles,
                      int* seg_start, int max_tiles, const int* idx_stm, const int* idx_nstm, const int* nnz, int A, int N,
                      int rows_per_slice, int n_persp, int* items, int* item_seg, int* hist);
int launch_ft_reduce_virtual(cudaStream_t s, float* grad, int N, int pi, int F);
int launch_ft_fold(cudaStream_t s, const float* w, void* comb, int N, int pi, int F, int half_comb = 0);
// dst[i] = fp16(src[i]) (cast_f32_to_f16, native_kernels.cu:648), n a multiple of 4
int launch_cast_half(cudaStream_t s, const float* src, void* dst, int64_t n);

// psv.cu
int launch_psv_extract(cudaStream_t s, int feature_set, const void* d_psv, long long n, int* stm, int* nstm, int* nnz,
                       int* bucket, float* score, float* wdl);
bool psv_feature_set_dims(int feature_set, int* ft_in, int* max_active);

// dense_kernels.cu
// tf32: run the contraction on the tensor cores with TF32 operands (l1_tc.cu) where the shape allows; error_flag: device
// int raised when one of that kernel's bounded waits ran out
int launch_l1_forward(cudaStream_t s, const float* x, int K, const int* order, const TileDesc* tiles,
                      const int* n_tiles, int max_tiles, const float* wb /*[nb][l1][K] or NULL*/,
                      const float* bb, const float* ws /*[K][l1]*/, const float* bs, float* y /*[B][l1]*/,
                      int l1, int nb, float* weff /*scratch [(nb + 1) * l1 * (K + 1)] or NULL*/, int tf32 = 0,
                      int* error_flag = nullptr);
// l1_tc.cu
bool l1_forward_tc_supported(int K, int l1);
int launch_l1_forward_tc(cudaStream_t s, const float* x, int K, const int* order, const TileDesc* tiles, const int* n_tiles,
                         int max_tiles, const float* weff, const float* beff, float* y, int l1, int nb, int* error_flag);
// sum over the batch of the extended WRM loss's per-position weights (wrm_weight_sum, native_kernels.cu:520-545), in a
// fixed order; partials: scratch of ceil(B / 256) doubles
int launch_wrm_weight_sum(cudaStream_t s, const float* score, int B, LossParams lp, double* partials, double* weight_sum);
int launch_tail_layerstack(cudaStream_t s, const float* l1_total, const int* bucket, const float* score,
                           const float* wdl, const float* l2_w, const float* l2_b, const float* l3_w,
                           const float* l3_b, LossParams lp, int B, int l1, int l2, int nb, float* net_output,
                           float* dy, float* dl1_total, float* l2_input, float* dl2_out, float* l2_acted,
                           double* loss_partials, double* loss_acc, int backward);
int launch_tail_simple(cudaStream_t s, const float* l1_pre, const float* score, const float* wdl,
                       const float* l2_w, const float* l2_b, const float* l3_w, const float* l3_b, LossParams lp,
                       int act, int B, int l1, int l2, float* net_output, float* dy, float* dl1_pre,
                       float* l1_acted, float* dl2_pre, float* l2_acted, double* loss_partials,
                       double* loss_acc, int backward);
// per-bucket reductions of the small layers: out[g][cell] = sum over the positions of bucket g
int launch_small_wgrad_layerstack(cudaStream_t s, const int* order, const int* seg_start, int B, int l1, int l2,
                                  int nb, const float* l2_input, const float* dl2_out, const float* l2_acted,
                                  const float* dy, const float* dl1_total, float* partials, float* l2_w_grad,
                                  float* l2_b_grad, float* l3_w_grad, float* l3_b_grad, float* l1_b_grad,
                                  float* l1s_b_grad);
int launch_small_wgrad_simple(cudaStream_t s, const int* order, const int* seg_start, int B, int l1, int l2,
                              const float* l1_acted, const float* dl2_pre, const float* l2_acted, const float* dy,
                              const float* dl1_pre, float* partials, float* l2_w_grad, float* l2_b_grad,
                              float* l3_w_grad, float* l3_b_grad, float* l1_b_grad);
// L1 weight gradient: LayerStack writes gw_bucket [nb][l1][K] and gw_shared [K][l1]; Simple only gw_shared.
int launch_l1_wgrad(cudaStream_t s, const float* x, int K, const float* dl1, const int* order,
                    const TileDesc* tiles, const int* n_tiles, int max_tiles, int l1, int nb, float* partials,
                    float* gw_bucket, float* gw_shared);
// L1 input gradient fused with the FT activation gradient; writes dft of both perspectives and the
// FT bias gradient.
// half_act: pre-activations and dft are fp16; dft is written as round(clamp(g * grad_scale)) and the clamped elements
// are added to *clamp_counter.  Returns -1 for a combination that is not built.
int launch_l1_dgrad_ftgrad(cudaStream_t s, int mode, const float* dl1, const int* order, const TileDesc* tiles,
                           const int* n_tiles, int max_tiles, const float* wb, const float* ws,
                           const void* pre_stm, const void* pre_nstm, const float* ft_bias, float scale,
                           int B, int F, int l1, int nb, void* dft_stm, void* dft_nstm, float* bias_partials,
                           float* ft_b_grad, int n_ctas, int half_act = 0, float grad_scale = 1.0f,
                           unsigned long long* clamp_counter = nullptr);

// opt_kernels.cu
// half_state: m and v are fp16 arrays (scaled, see above); mirror: NULL or an fp16 copy of the updated weights
int launch_radam(cudaStream_t s, float* w, void* m, void* v, const float* g, float* slow, int64_t n,
                 OptScalars sc, int half_state = 0, void* mirror = nullptr);
int launch_radam_small(cudaStream_t s, const SmallGroups& groups, int max_n, OptScalars sc);
// factorised FT table: per virtual row v, updates the real rows kb*pi+v, reduces their gradients into the
// virtual row, updates it and writes the folded forward table.
// the same in pieces: the real rows of the king buckets [kb0, kb1) (call with ascending ranges), then the virtual rows
// and the folded table
// half_state: m and v are fp16 (scaled); half_comb: the folded table is fp16 (ft_fold_virtual_f16, native_kernels.cu:262)
int launch_radam_factorized_rows(cudaStream_t s, float* w, void* m, void* v, float* g, float* slow, int N, int pi, int F, int kb0,
                                 int kb1, OptScalars sc, int half_state = 0);
int launch_radam_factorized_fold(cudaStream_t s, float* w, void* m, void* v, float* g, float* slow, void* comb, int N, int pi,
                                 int F, OptScalars sc, int half_state = 0, int half_comb = 0);
int launch_radam_factorized(cudaStream_t s, float* w, void* m, void* v, float* g, float* slow, void* comb,
                            int N, int pi, int F, OptScalars sc, int half_state = 0, int half_comb = 0);
