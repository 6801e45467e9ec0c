/*
 * CPU oracle for the NNUE training step — TEST INFRASTRUCTURE, not product code.
 * See tatara_oracle.h for scope and parity status.  Every function cites the
 * reference file it restates (paths relative to the reference project root).
 * Loop order and f32/f64 types follow the reference so that sums round the
 * same way.  OpenMP pragmas only split loops whose iterations write disjoint
 * outputs, so results do not depend on the thread count.
 */
#include "tatara_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 1;
#define PAR_FOR _Pragma("omp parallel for schedule(static) num_threads(g_threads) if (g_threads > 1)")

/* ================================================================================
 * sparse feature transformer
 * ================================================================================ */

/* crates/gpu-kernels/src/sparse/sparse_ft_forward.rs:54-78 */
void ora_sparse_ft_forward(const float* weight, const int32_t* indices, const int32_t* nnz_arr,
                           float* out, size_t batch, size_t rows, size_t cols, size_t max_active) {
    PAR_FOR
    for (size_t bi = 0; bi < batch; ++bi) {
        for (size_t ri = 0; ri < rows; ++ri) {
            float sum = 0.0f;
            for (size_t ni = 0; ni < (size_t)nnz_arr[bi]; ++ni) {
                int32_t idx = indices[bi * max_active + ni];
                if (idx >= 0 && (size_t)idx < cols) sum += weight[(size_t)idx * rows + ri];
            }
            out[bi * rows + ri] = sum;
        }
    }
}

/* crates/gpu-kernels/src/sparse/sparse_ft_backward.rs:51-73 (accumulates; scans all nnz slots) */
void ora_sparse_ft_backward(const float* grad_out, const int32_t* indices, float* grad_weight,
                            size_t batch, size_t rows, size_t cols, size_t nnz) {
    /* threads own disjoint column ranges; per cell the adds stay in bi order */
    PAR_FOR
    for (size_t ri = 0; ri < rows; ++ri) {
        for (size_t bi = 0; bi < batch; ++bi) {
            float g = grad_out[bi * rows + ri];
            for (size_t ni = 0; ni < nnz; ++ni) {
                int32_t idx = indices[bi * nnz + ni];
                if (idx >= 0 && (size_t)idx < cols) grad_weight[(size_t)idx * rows + ri] += g;
            }
        }
    }
}

/* crates/gpu-kernels/src/sparse/ft_factorize.rs:78-99, base mode (virtual row = feature % pi) */
void ora_ft_fold_virtual(const float* w, float* comb, size_t ft_in, size_t ft_out, size_t piece_inputs) {
    PAR_FOR
    for (size_t feature = 0; feature < ft_in; ++feature) {
        size_t vrow = feature % piece_inputs;
        for (size_t ri = 0; ri < ft_out; ++ri)
            comb[feature * ft_out + ri] = w[feature * ft_out + ri] + w[(ft_in + vrow) * ft_out + ri];
    }
}

/* crates/gpu-kernels/src/sparse/ft_factorize.rs:109-121, base mode */
void ora_ft_reduce_virtual_grad(float* grad, size_t ft_in, size_t ft_out, size_t piece_inputs) {
    PAR_FOR
    for (size_t vrow = 0; vrow < piece_inputs; ++vrow) {
        for (size_t ri = 0; ri < ft_out; ++ri) {
            float sum = 0.0f;
            for (size_t feature = vrow; feature < ft_in; feature += piece_inputs)
                sum += grad[feature * ft_out + ri];
            grad[(ft_in + vrow) * ft_out + ri] = sum;
        }
    }
}

/* ================================================================================
 * LayerStack pieces
 * ================================================================================ */

/* crates/gpu-kernels/src/layerstack/ft_post_perspective.rs:42-51 */
static inline float crelu01(float x) { return x < 0.0f ? 0.0f : (x > 1.0f ? 1.0f : x); }

/* ft_post_perspective.rs:57-83 */
void ora_ft_post_perspective_fwd(const float* stm, const float* nstm, const float* bias,
                                 float* combined, size_t batch, size_t ft_dim, float scale) {
    size_t half = ft_dim / 2;
    PAR_FOR
    for (size_t bi = 0; bi < batch; ++bi) {
        size_t base = bi * ft_dim;
        for (size_t ri = 0; ri < ft_dim; ++ri) {
            float val;
            if (ri < half) {
                float xa = stm[base + ri] + bias[ri];
                float xb = stm[base + half + ri] + bias[half + ri];
                val = crelu01(xa) * crelu01(xb) * scale;
            } else {
                size_t p = ri - half;
                float xa = nstm[base + p] + bias[p];
                float xb = nstm[base + half + p] + bias[half + p];
                val = crelu01(xa) * crelu01(xb) * scale;
            }
            combined[bi * ft_dim + ri] = val;
        }
    }
}

/* ft_post_perspective.rs:92-129 (grad_bias accumulates) */
void ora_ft_post_perspective_grad(const float* d_combined, const float* ft_out, const float* bias,
                                  float* grad_ft_out, float* grad_bias, size_t batch, size_t ft_dim,
                                  size_t d_combined_offset, size_t d_combined_stride, float scale) {
    size_t half = ft_dim / 2;
    /* column-parallel so that grad_bias[ii] keeps its bi order */
    PAR_FOR
    for (size_t ii = 0; ii < ft_dim; ++ii) {
        size_t pair = ii < half ? ii : ii - half;
        int is_first = ii < half;
        for (size_t bi = 0; bi < batch; ++bi) {
            size_t base = bi * ft_dim;
            float dy = d_combined[bi * d_combined_stride + d_combined_offset + pair];
            float xa = ft_out[base + pair] + bias[pair];
            float xb = ft_out[base + half + pair] + bias[half + pair];
            float ya = crelu01(xa), yb = crelu01(xb);
            float my_pre = is_first ? xa : xb;
            float partner_post = is_first ? yb : ya;
            float g_post = dy * partner_post * scale;
            float g_pre = (my_pre > 0.0f && my_pre < 1.0f) ? g_post : 0.0f;
            grad_ft_out[base + ii] = g_pre;
            grad_bias[ii] += g_pre;
        }
    }
}

/* crates/gpu-kernels/src/layerstack/dense_mm.rs:37-54 — w is [in_dim, out_dim] */
void ora_dense_mm_fwd(const float* x, const float* w, const float* bias, float* y,
                      size_t batch, size_t in_dim, size_t out_dim) {
    PAR_FOR
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t oi = 0; oi < out_dim; ++oi) {
            float sum = bias[oi];
            for (size_t k = 0; k < in_dim; ++k) sum += x[bi * in_dim + k] * w[k * out_dim + oi];
            y[bi * out_dim + oi] = sum;
        }
}

/* dense_mm.rs:56-73 */
void ora_dense_mm_bwd_input(const float* dy, const float* w, float* dx,
                            size_t batch, size_t in_dim, size_t out_dim) {
    PAR_FOR
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t ii = 0; ii < in_dim; ++ii) {
            float sum = 0.0f;
            for (size_t o = 0; o < out_dim; ++o) sum += dy[bi * out_dim + o] * w[ii * out_dim + o];
            dx[bi * in_dim + ii] = sum;
        }
}

/* dense_mm.rs:75-92 (overwrites) */
void ora_dense_mm_bwd_weight(const float* x, const float* dy, float* grad_w,
                             size_t batch, size_t in_dim, size_t out_dim) {
    PAR_FOR
    for (size_t ii = 0; ii < in_dim; ++ii)
        for (size_t oi = 0; oi < out_dim; ++oi) {
            float sum = 0.0f;
            for (size_t b = 0; b < batch; ++b) sum += x[b * in_dim + ii] * dy[b * out_dim + oi];
            grad_w[ii * out_dim + oi] = sum;
        }
}

/* dense_mm.rs:94-100 (accumulates) */
void ora_bias_grad(const float* dy, float* grad_bias, size_t batch, size_t out_dim) {
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t oi = 0; oi < out_dim; ++oi) grad_bias[oi] += dy[bi * out_dim + oi];
}

/* crates/gpu-kernels/src/layerstack/dense_mm_bucket.rs:45-73 — w is [nb, out_dim, in_dim] */
void ora_dense_mm_fwd_bucket(const float* x, const float* w, const float* bias, const int32_t* bucket_idx,
                             float* y, size_t batch, size_t in_dim, size_t out_dim, size_t num_buckets) {
    PAR_FOR
    for (size_t bi = 0; bi < batch; ++bi) {
        int32_t buc = bucket_idx[bi];
        if (buc < 0 || (size_t)buc >= num_buckets) {
            for (size_t oi = 0; oi < out_dim; ++oi) y[bi * out_dim + oi] = 0.0f;
            continue;
        }
        size_t g = (size_t)buc;
        for (size_t oi = 0; oi < out_dim; ++oi) {
            size_t wb = g * out_dim * in_dim + oi * in_dim;
            float sum = bias[g * out_dim + oi];
            for (size_t k = 0; k < in_dim; ++k) sum += x[bi * in_dim + k] * w[wb + k];
            y[bi * out_dim + oi] = sum;
        }
    }
}

/* dense_mm_bucket.rs:79-106 */
void ora_dense_mm_bwd_input_bucket(const float* dy, const float* w, const int32_t* bucket_idx, float* dx,
                                   size_t batch, size_t in_dim, size_t out_dim, size_t num_buckets) {
    PAR_FOR
    for (size_t bi = 0; bi < batch; ++bi) {
        int32_t buc = bucket_idx[bi];
        if (buc < 0 || (size_t)buc >= num_buckets) {
            for (size_t ii = 0; ii < in_dim; ++ii) dx[bi * in_dim + ii] = 0.0f;
            continue;
        }
        size_t g = (size_t)buc;
        for (size_t ii = 0; ii < in_dim; ++ii) {
            float sum = 0.0f;
            for (size_t o = 0; o < out_dim; ++o)
                sum += dy[bi * out_dim + o] * w[g * out_dim * in_dim + o * in_dim + ii];
            dx[bi * in_dim + ii] = sum;
        }
    }
}

/* dense_mm_bucket.rs:112-135 (overwrites) */
void ora_dense_mm_bwd_weight_bucket(const float* x, const float* dy, const int32_t* bucket_idx,
                                    float* grad_w, size_t batch, size_t in_dim, size_t out_dim,
                                    size_t num_buckets) {
    size_t per_bucket = out_dim * in_dim;
    size_t cells = num_buckets * per_bucket;
    PAR_FOR
    for (size_t cell = 0; cell < cells; ++cell) {
        size_t g = cell / per_bucket, rem = cell % per_bucket;
        size_t oi = rem / in_dim, ii = rem % in_dim;
        int32_t target = (int32_t)g;
        float sum = 0.0f;
        for (size_t b = 0; b < batch; ++b)
            if (bucket_idx[b] == target) sum += x[b * in_dim + ii] * dy[b * out_dim + oi];
        grad_w[cell] = sum;
    }
}

/* dense_mm_bucket.rs:141-161 (accumulates) */
void ora_bias_grad_bucket(const float* dy, const int32_t* bucket_idx, float* grad_bias,
                          size_t batch, size_t out_dim, size_t num_buckets) {
    for (size_t bi = 0; bi < batch; ++bi) {
        int32_t buc = bucket_idx[bi];
        if (buc < 0 || (size_t)buc >= num_buckets) continue;
        for (size_t oi = 0; oi < out_dim; ++oi) grad_bias[(size_t)buc * out_dim + oi] += dy[bi * out_dim + oi];
    }
}

/* crates/gpu-kernels/src/layerstack/crelu.rs */
void ora_crelu_fwd(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = crelu01(x[i]);
}
void ora_crelu_grad(const float* x, const float* dy, float* dx, size_t n) {
    for (size_t i = 0; i < n; ++i) dx[i] = (x[i] > 0.0f && x[i] < 1.0f) ? dy[i] : 0.0f;
}
/* crates/gpu-kernels/src/pointwise/screlu_fwd.rs, screlu_grad.rs */
void ora_screlu_fwd(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; ++i) { float a = crelu01(x[i]); y[i] = a * a; }
}
void ora_screlu_grad(const float* x, const float* dy, float* dx, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float a = x[i];
        if (a < 0.0f) a = 0.0f;
        if (a > 1.0f) a = 1.0f; /* f32::clamp keeps NaN */
        float d = (a > 0.0f && a < 1.0f) ? 2.0f * a : 0.0f;
        dx[i] = dy[i] * d;
    }
}
/* crates/gpu-kernels/src/layerstack/abs_pow2_scale.rs */
void ora_abs_pow2_scale_fwd(const float* x, float* y, float scale, size_t n) {
    for (size_t i = 0; i < n; ++i) y[i] = x[i] * x[i] * scale;
}
void ora_abs_pow2_scale_grad(const float* x, const float* dy, float* dx, float scale, size_t n) {
    for (size_t i = 0; i < n; ++i) dx[i] = 2.0f * x[i] * scale * dy[i];
}
/* crates/gpu-kernels/src/layerstack/concat_l1sqr_main.rs */
void ora_concat_l1sqr_main_fwd(const float* a, const float* b, float* out, size_t batch, size_t a_dim, size_t b_dim) {
    size_t od = a_dim + b_dim;
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t oi = 0; oi < od; ++oi)
            out[bi * od + oi] = oi < a_dim ? a[bi * a_dim + oi] : b[bi * b_dim + (oi - a_dim)];
}
void ora_concat_l1sqr_main_grad(const float* dout, float* da, float* db, size_t batch, size_t dim) {
    size_t od = 2 * dim;
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t ii = 0; ii < dim; ++ii) {
            da[bi * dim + ii] = dout[bi * od + ii];
            db[bi * dim + ii] = dout[bi * od + dim + ii];
        }
}
/* crates/gpu-kernels/src/layerstack/slice2d.rs */
void ora_slice_extract_2d(const float* src, float* dst, size_t batch, size_t src_stride, size_t src_offset, size_t out_dim) {
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t oi = 0; oi < out_dim; ++oi) dst[bi * out_dim + oi] = src[bi * src_stride + src_offset + oi];
}
void ora_slice_scatter_2d(const float* src, float* dst, size_t batch, size_t in_dim, size_t dst_stride, size_t dst_offset) {
    for (size_t bi = 0; bi < batch; ++bi)
        for (size_t ii = 0; ii < in_dim; ++ii) dst[bi * dst_stride + dst_offset + ii] = src[bi * in_dim + ii];
}
/* crates/gpu-kernels/src/layerstack/elementwise.rs */
void ora_elementwise_add(const float* a, const float* b, float* c, size_t n) {
    for (size_t i = 0; i < n; ++i) c[i] = a[i] + b[i];
}

/* ================================================================================
 * losses
 * ================================================================================ */
static inline float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

/* crates/gpu-kernels/src/pointwise/loss_wdl.rs:63-88 */
void ora_loss_wdl(const float* out, const float* score, const float* wdl, const float* per_pos_norm,
                  float* dl_dout, double* loss_acc, float lambda, float scale, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float p = sigmoid_f32(out[i] * scale);
        float ys = sigmoid_f32(score[i] * scale);
        float y = lambda * wdl[i] + (1.0f - lambda) * ys;
        float err = p - y;
        float norm = per_pos_norm[i];
        *loss_acc += (double)err * (double)err;
        dl_dout[i] = 2.0f * err * p * (1.0f - p) * scale * norm;
    }
}

/* crates/gpu-kernels/src/pointwise/loss_wrm.rs:182-194 */
static float wrm_weight(float score, float target_offset, float target_scaling, float w1, float w2) {
    float pt = (score - target_offset) / target_scaling;
    float pmt = (-score - target_offset) / target_scaling;
    float pf = 0.5f * (1.0f + sigmoid_f32(pt) - sigmoid_f32(pmt));
    float wb = (pf - 0.5f) * (pf - 0.5f) * pf * (1.0f - pf);
    return 1.0f + (powf(2.0f, w1) - 1.0f) * powf(wb, w2);
}

/* crates/gpu-kernels/src/pointwise/loss_wrm.rs:99-180 */
void ora_loss_wrm(const float* out, const float* score, const float* wdl, const float* per_pos_norm,
                  float* dl_dout, double* loss_acc, float lambda, float nnue2score, float in_scaling,
                  float in_offset, float target_offset, float target_scaling, float pow_exp,
                  float qp_asymmetry, float weight_boost_w1, float weight_boost_w2, int extended, size_t n) {
    float inv_sum_w = 0.0f;
    if (extended) {
        double sum_w = 0.0;
        for (size_t i = 0; i < n; ++i)
            sum_w += (double)wrm_weight(score[i], target_offset, target_scaling, weight_boost_w1, weight_boost_w2);
        inv_sum_w = (float)(1.0 / sum_w);
    }
    for (size_t i = 0; i < n; ++i) {
        float s = score[i];
        float pt = (s - target_offset) / target_scaling;
        float pmt = (-s - target_offset) / target_scaling;
        float target_wrm = 0.5f * (1.0f + sigmoid_f32(pt) - sigmoid_f32(pmt));
        float target = lambda * wdl[i] + (1.0f - lambda) * target_wrm;
        float scorenet = out[i] * nnue2score;
        float q = sigmoid_f32((scorenet - in_offset) / in_scaling);
        float qm = sigmoid_f32((-scorenet - in_offset) / in_scaling);
        float qf = 0.5f * (1.0f + q - qm);
        float err = qf - target;
        if (!extended) {
            float norm = per_pos_norm[i];
            *loss_acc += (double)err * (double)err;
            dl_dout[i] = err * (nnue2score / in_scaling) * (q * (1.0f - q) + qm * (1.0f - qm)) * norm;
            continue;
        }
        float pf = target_wrm;
        float wb = (pf - 0.5f) * (pf - 0.5f) * pf * (1.0f - pf);
        float weight = 1.0f + (powf(2.0f, weight_boost_w1) - 1.0f) * powf(wb, weight_boost_w2);
        float asym = qf > target ? 1.0f + qp_asymmetry : 1.0f;
        float abs_err = fabsf(err);
        float pow_abs = powf(abs_err, pow_exp - 1.0f);
        float signed_pow = err < 0.0f ? -pow_abs : pow_abs;
        float dqf = 0.5f * (nnue2score / in_scaling) * (q * (1.0f - q) + qm * (1.0f - qm));
        dl_dout[i] = (weight * inv_sum_w) * (asym * pow_exp * signed_pow) * dqf;
        float loss_i = asym * powf(abs_err, pow_exp) * weight * (float)n * inv_sum_w;
        *loss_acc += (double)loss_i;
    }
}

/* ================================================================================
 * optimizer
 * ================================================================================ */

/* crates/gpu-kernels/src/pointwise/radam_step.rs:63-86 */
void ora_radam_compute_step_size_denom(uint64_t step, float beta1, float beta2, float n_sma_threshold,
                                       float* step_size, int32_t* denom) {
    float step_f = (float)step;
    float beta2_t = powf(beta2, step_f);
    float n_sma_max = 2.0f / (1.0f - beta2) - 1.0f;
    float n_sma = n_sma_max - 2.0f * step_f * beta2_t / (1.0f - beta2_t);
    float bc1 = 1.0f - powf(beta1, step_f);
    if (n_sma > n_sma_threshold) {
        float p1 = (n_sma - 4.0f) / (n_sma_max - 4.0f);
        float p2 = (n_sma - 2.0f) / n_sma;
        float p3 = n_sma_max / (n_sma_max - 2.0f);
        *step_size = sqrtf((1.0f - beta2_t) * p1 * p2 * p3) / bc1;
    } else {
        *step_size = 1.0f / bc1;
    }
    *denom = n_sma > n_sma_threshold ? 1 : 0;
}

/* radam_step.rs:116-156 */
void ora_radam_step(float* weights, float* m, float* v, float* grad, float lr, float step_size,
                    int32_t denom, float decay, float beta1, float beta2, float eps,
                    float min_w, float max_w, size_t n) {
    float rate = lr * step_size;
    PAR_FOR
    for (size_t i = 0; i < n; ++i) {
        float g = grad[i];
        float p = weights[i];
        p *= 1.0f - decay * rate;
        float mi = beta1 * m[i] + (1.0f - beta1) * g;
        float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
        m[i] = mi;
        v[i] = vi;
        float val = mi;
        if (denom != 0) val /= sqrtf(vi) + eps;
        p -= rate * val;
        if (p < min_w) p = min_w;
        if (p > max_w) p = max_w;
        weights[i] = p;
        grad[i] = 0.0f;
    }
}

/* ---- reduced precision (--ft-fp16, --ft-fp16-out, --fp16-opt-state, --tf32) ------------------------------------------
 * The reference has no CPU twin for these modes; the functions below restate its CUDA kernels
 * (crates/cuda-native-runtime/kernels/native_kernels.cu) with their rounding points.  fp16 values are kept in float
 * arrays holding exactly representable fp16 values. */
float ora_round_half(float x) { return (float)(_Float16)x; } /* __float2half_rn followed by __half2float */

/* TF32 operand: cuBLAS in CUBLAS_TF32_TENSOR_OP_MATH (bins/nnue_train/src/trainer_common.rs:691-727) feeds fp32 data to
 * the tensor cores, which read the sign, the exponent and the upper 10 mantissa bits.  Modelled as truncation. */
float ora_tf32(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    u &= 0xFFFFE000u;
    memcpy(&x, &u, 4);
    return x;
}

/* native_clamp_half, native_kernels.cu:636-646 */
static float clamp_half_count(float v, uint64_t* clamps) {
    if (v > 65504.0f) { ++*clamps; return 65504.0f; }
    if (v < -65504.0f) { ++*clamps; return -65504.0f; }
    return v;
}

/* native_radam_step_fp16<HalfState = true>, native_kernels.cu:1127-1181.  m and v hold the stored fp16 values divided by
 * their scale (what MomentBuf::to_host_f32 returns, bins/nnue_train/src/trainer_common.rs:89-105). */
void ora_radam_step_f16state(float* weights, float* m, float* v, float* grad, float lr, float step_size, int32_t denom,
                             float decay, float beta1, float beta2, float eps, float min_w, float max_w, float m_scale,
                             float v_scale, size_t n) {
    float rate = lr * step_size;
    PAR_FOR
    for (size_t i = 0; i < n; ++i) {
        float g = grad[i];
        float p = weights[i] * (1.0f - decay * rate);
        float prev_m = m[i], prev_v = v[i]; /* = half2float(stored) / scale */
        float mi = beta1 * prev_m + (1.0f - beta1) * g;
        float vi = beta2 * prev_v + (1.0f - beta2) * g * g;
        float sm = mi * m_scale;
        sm = sm > 65504.0f ? 65504.0f : (sm < -65504.0f ? -65504.0f : sm);
        float sv = vi * v_scale;
        sv = sv > 65504.0f ? 65504.0f : sv;
        m[i] = ora_round_half(sm) / m_scale;
        v[i] = ora_round_half(sv) / v_scale;
        float val = mi;
        if (denom != 0) val /= sqrtf(vi) + eps;
        p -= rate * val;
        p = p < min_w ? min_w : (p > max_w ? max_w : p);
        weights[i] = p;
        grad[i] = 0.0f;
    }
}

/* crates/gpu-kernels/src/pointwise/ranger_step.rs:52-59 */
void ora_ranger_lookahead_lerp(float* weights, float* slow, float alpha, size_t n) {
    float oma = 1.0f - alpha;
    PAR_FOR
    for (size_t i = 0; i < n; ++i) {
        float nw = alpha * weights[i] + oma * slow[i];
        weights[i] = nw;
        slow[i] = nw;
    }
}

/* crates/nnue-train/src/optimizer.rs:63-93 */
void ora_optimizer_scalars(int kind, uint64_t step, float beta2, float n_sma_threshold,
                           float* step_size, int32_t* denom, float* beta1) {
    float b1 = kind == 0 ? 0.99f : 0.9f;
    *beta1 = b1;
    if (kind == 2) { *step_size = 1.0f; *denom = 1; return; }
    ora_radam_compute_step_size_denom(step, b1, beta2, n_sma_threshold, step_size, denom);
}

/* ================================================================================
 * weight init — crates/nnue-train/src/init.rs:111-210
 * ================================================================================ */
static inline float xs_next_unit(uint64_t* s) {
    *s ^= *s << 13;
    *s ^= *s >> 7;
    *s ^= *s << 17;
    return (float)(*s >> 11) / (float)(1ull << 53);
}

void ora_init_sample(float* out, size_t n, size_t num_buckets, size_t fan_in, int dist,
                     int scale_kind, float scale_value, int per_bucket_repeat, uint64_t seed) {
    if (dist == 0) { memset(out, 0, n * sizeof(float)); return; }
    float mag;
    if (scale_kind == 0) mag = scale_value;
    else { float f = (float)(fan_in < 1 ? 1 : fan_in); mag = sqrtf(scale_value / f); }
    size_t block_len = per_bucket_repeat ? n / num_buckets : n;
    uint64_t s = seed < 1 ? 1 : seed;
    for (size_t i = 0; i < block_len; ++i) out[i] = (xs_next_unit(&s) * 2.0f - 1.0f) * mag;
    if (per_bucket_repeat && num_buckets > 1)
        for (size_t g = 1; g < num_buckets; ++g) memcpy(out + g * block_len, out, block_len * sizeof(float));
}

/* ================================================================================
 * PackedSfenValue decode — crates/shogi-format/src/packed_sfen.rs
 * ================================================================================ */
enum { PT_NONE = 0, PT_PAWN, PT_LANCE, PT_KNIGHT, PT_SILVER, PT_BISHOP, PT_ROOK, PT_GOLD, PT_KING,
       PT_PRO_PAWN, PT_PRO_LANCE, PT_PRO_KNIGHT, PT_PRO_SILVER, PT_HORSE, PT_DRAGON };

/* packed_sfen.rs:26-35: (pattern, bits), LSB first; index = huffman piece id */
static const uint8_t HUFF_PATTERN[8] = {0x00, 0x01, 0x03, 0x0b, 0x07, 0x1f, 0x3f, 0x0f};
static const uint8_t HUFF_BITS[8] = {1, 2, 4, 4, 4, 6, 6, 5};
/* huffman id -> PieceType (packed_sfen.rs:559-570): none,pawn,lance,knight,silver,bishop,rook,gold */
static const uint8_t HUFF_PT[8] = {PT_NONE, PT_PAWN, PT_LANCE, PT_KNIGHT, PT_SILVER, PT_BISHOP, PT_ROOK, PT_GOLD};
#define HUFF_GOLD 7

typedef struct { const uint8_t* data; size_t cursor, limit; } bitstream;

static int bs_read_bit(bitstream* s) {
    if (s->cursor >= s->limit) return 0;
    int bit = (s->data[s->cursor / 8] >> (s->cursor % 8)) & 1;
    s->cursor++;
    return bit;
}
static uint32_t bs_read_bits(bitstream* s, int n) {
    uint32_t r = 0;
    for (int i = 0; i < n; ++i) if (bs_read_bit(s)) r |= 1u << i;
    return r;
}
/* packed_sfen.rs:153-168: bits past the end read as 0 */
static uint32_t bs_peek_bits(const bitstream* s, int n) {
    uint32_t r = 0;
    for (int i = 0; i < n; ++i) {
        size_t c = s->cursor + (size_t)i;
        if (c < s->limit && ((s->data[c / 8] >> (c % 8)) & 1)) r |= 1u << i;
    }
    return r;
}
/* packed_sfen.rs:66-110: first table entry whose (shortened, for hand) pattern matches the peeked bits */
static int huff_match(uint32_t peek, int hand, int* code_bits) {
    for (int i = 0; i < 8; ++i) {
        if (hand && i == 0) continue;
        uint32_t pattern = HUFF_PATTERN[i];
        int len = HUFF_BITS[i];
        if (hand) { pattern >>= 1; len -= 1; }
        uint32_t mask = (1u << len) - 1;
        if ((peek & mask) == pattern) { *code_bits = len; return i; }
    }
    *code_bits = 0;
    return 0;
}
static uint8_t promote_pt(uint8_t pt) {
    switch (pt) {
        case PT_PAWN: return PT_PRO_PAWN;
        case PT_LANCE: return PT_PRO_LANCE;
        case PT_KNIGHT: return PT_PRO_KNIGHT;
        case PT_SILVER: return PT_PRO_SILVER;
        case PT_BISHOP: return PT_HORSE;
        case PT_ROOK: return PT_DRAGON;
        default: return pt;
    }
}
static int hand_slot(uint8_t pt) { /* types.rs Hand::piece_index */
    switch (pt) {
        case PT_PAWN: return 0; case PT_LANCE: return 1; case PT_KNIGHT: return 2; case PT_SILVER: return 3;
        case PT_GOLD: return 4; case PT_BISHOP: return 5; case PT_ROOK: return 6; default: return -1;
    }
}

/* packed_sfen.rs:387-448 */
void ora_psv_decode(const uint8_t* psv, ora_board* b) {
    memset(b, 0, sizeof(*b));
    b->score = (int16_t)((uint16_t)psv[32] | ((uint16_t)psv[33] << 8));
    b->ply = (uint16_t)((uint16_t)psv[36] | ((uint16_t)psv[37] << 8));
    b->result = (int8_t)psv[38];
    bitstream s = {psv, 0, 256};
    b->side_to_move = (uint8_t)bs_read_bit(&s);
    uint8_t bk = (uint8_t)bs_read_bits(&s, 7), wk = (uint8_t)bs_read_bits(&s, 7);
    b->black_king_sq = bk;
    b->white_king_sq = wk;
    if (bk < 81) { b->board_pt[bk] = PT_KING; b->board_color[bk] = 0; }
    if (wk < 81) { b->board_pt[wk] = PT_KING; b->board_color[wk] = 1; }
    for (int sq = 0; sq < 81; ++sq) {
        if (sq == bk || sq == wk) continue;
        int bits;
        int id = huff_match(bs_peek_bits(&s, 6), 0, &bits);
        s.cursor += (size_t)bits;
        if (id == 0) { b->board_pt[sq] = PT_NONE; b->board_color[sq] = 0; continue; }
        int promoted = id != HUFF_GOLD ? bs_read_bit(&s) : 0;
        int color = bs_read_bit(&s);
        uint8_t pt = HUFF_PT[id];
        b->board_pt[sq] = promoted ? promote_pt(pt) : pt;
        b->board_color[sq] = (uint8_t)color;
    }
    while (s.cursor < 256) {
        int bits;
        int id = huff_match(bs_peek_bits(&s, 5), 1, &bits);
        s.cursor += (size_t)bits;
        int piecebox = id != HUFF_GOLD ? bs_read_bit(&s) : 0;
        int color = bs_read_bit(&s);
        if (piecebox) continue;
        int slot = hand_slot(HUFF_PT[id]);
        if (slot >= 0) b->hand[color][slot]++;
    }
}

/* ================================================================================
 * BonaPiece + feature sets — crates/shogi-format/src/bona_piece.rs,
 * crates/shogi-features/src/feature_set.rs
 * ================================================================================ */
#define FE_HAND_END 90
#define F_KING 1548
#define E_KING 1629
/* bona_piece.rs:59-90: [piece type][is_friend] */
static const uint16_t PIECE_BASE[15][2] = {
    {0, 0}, {171, 90}, {333, 252}, {495, 414}, {657, 576}, {981, 900}, {1305, 1224}, {819, 738},
    {0, 0}, {819, 738}, {819, 738}, {819, 738}, {819, 738}, {1143, 1062}, {1467, 1386}};
/* bona_piece.rs:13-30: hand bases [slot][is_friend] in HAND_PIECE_TYPES order */
static const uint16_t HAND_BASE[7][2] = {{20, 1}, {44, 39}, {54, 49}, {64, 59}, {74, 69}, {82, 79}, {88, 85}};
/* types.rs:271-285 */
static const uint8_t BOARD_PIECE_TYPES[13] = {PT_PAWN, PT_LANCE, PT_KNIGHT, PT_SILVER, PT_GOLD, PT_BISHOP, PT_ROOK,
                                              PT_PRO_PAWN, PT_PRO_LANCE, PT_PRO_KNIGHT, PT_PRO_SILVER, PT_HORSE, PT_DRAGON};

typedef struct { int kings; /* 0 none, 1 split, 2 merged */ int mirror; int king_buckets, piece_inputs, max_active; } fs_spec;
static int fs_get(int feature_set, fs_spec* s) { /* feature_set.rs:1031-1038 */
    switch (feature_set) {
        case 0: *s = (fs_spec){0, 0, 81, 1548, 38}; return 0;
        case 1: *s = (fs_spec){1, 0, 81, 1710, 40}; return 0;
        case 2: *s = (fs_spec){2, 0, 81, 1629, 40}; return 0;
        case 3: *s = (fs_spec){1, 1, 45, 1710, 40}; return 0;
        case 4: *s = (fs_spec){2, 1, 45, 1629, 40}; return 0;
        default: return -1;
    }
}
int ora_feature_dims(int feature_set, int* king_buckets, int* piece_inputs, int* ft_in, int* max_active) {
    fs_spec s;
    if (fs_get(feature_set, &s)) return -1;
    *king_buckets = s.king_buckets; *piece_inputs = s.piece_inputs;
    *ft_in = s.king_buckets * s.piece_inputs; *max_active = s.max_active;
    return 0;
}
static inline int persp_index(int sq, int perspective) { return perspective == 0 ? sq : 80 - sq; }

/* bona_piece.rs:141-170 */
static int bp_from_piece_square(int pt, int color, int sq, int perspective) {
    if (pt == PT_NONE || pt == PT_KING) return 0;
    return PIECE_BASE[pt][color == perspective] + persp_index(sq, perspective);
}
/* bona_piece.rs:172-244 */
static int bp_from_hand(int perspective, int owner, int slot, int count) {
    if (count == 0) return 0;
    return HAND_BASE[slot][owner == perspective] + count - 1;
}
typedef struct { int king_bucket, mirror; } persp_ctx;
/* feature_set.rs:822-840 */
static persp_ctx make_ctx(const fs_spec* s, int king_sq, int perspective) {
    int k = persp_index(king_sq, perspective);
    persp_ctx c;
    if (!s->mirror) { c.king_bucket = k; c.mirror = 0; return c; }
    int file = k / 9, rank = k % 9;
    int fm = file >= 5 ? 8 - file : file;
    c.king_bucket = fm * 9 + rank;
    c.mirror = file >= 5;
    return c;
}
/* feature_set.rs:972-991 + :842-845 */
static int fs_index(const fs_spec* s, const persp_ctx* c, int bp) {
    int pp = bp;
    if (c->mirror && pp >= FE_HAND_END) {
        int rel = pp - FE_HAND_END;
        int piece_index = rel / 81, sq = rel % 81;
        int file = sq / 9, rank = sq % 9;
        pp = FE_HAND_END + piece_index * 81 + (8 - file) * 9 + rank;
    }
    if (s->kings == 2 && pp >= E_KING) pp -= 81;
    return c->king_bucket * s->piece_inputs + pp;
}

/* feature_set.rs:655-808 (base path); emission order of packed_sfen.rs:493-535 */
int ora_extract_active_features(int feature_set, const ora_board* b, int32_t* stm_out, int32_t* nstm_out, int cap) {
    fs_spec s;
    if (fs_get(feature_set, &s)) return -1;
    int stm = b->side_to_move, nstm = stm ^ 1;
    int stm_king = stm == 0 ? b->black_king_sq : b->white_king_sq;
    int nstm_king = nstm == 0 ? b->black_king_sq : b->white_king_sq;
    if (stm_king >= 81 || nstm_king >= 81) return 0;
    persp_ctx sc = make_ctx(&s, stm_king, stm), nc = make_ctx(&s, nstm_king, nstm);
    int count = 0;
    for (int t = 0; t < 13; ++t) {
        int pt = BOARD_PIECE_TYPES[t];
        for (int color = 0; color < 2; ++color)
            for (int sq = 0; sq < 81; ++sq) {
                if (b->board_pt[sq] != pt || b->board_color[sq] != color) continue;
                if (count >= cap) continue;
                stm_out[count] = fs_index(&s, &sc, bp_from_piece_square(pt, color, sq, stm));
                nstm_out[count] = fs_index(&s, &nc, bp_from_piece_square(pt, color, sq, nstm));
                count++;
            }
    }
    if (s.kings != 0) {
        if (count < cap) {
            stm_out[count] = fs_index(&s, &sc, F_KING + persp_index(stm_king, stm));
            nstm_out[count] = fs_index(&s, &nc, F_KING + persp_index(nstm_king, nstm));
            count++;
        }
        if (count < cap) {
            stm_out[count] = fs_index(&s, &sc, E_KING + persp_index(nstm_king, stm));
            nstm_out[count] = fs_index(&s, &nc, E_KING + persp_index(stm_king, nstm));
            count++;
        }
    }
    for (int owner = 0; owner < 2; ++owner)
        for (int slot = 0; slot < 7; ++slot) {
            int n_hand = b->hand[owner][slot];
            for (int i = 1; i <= n_hand; ++i) {
                if (count >= cap) return count;
                int sbp = bp_from_hand(stm, owner, slot, i);
                if (sbp != 0) {
                    stm_out[count] = fs_index(&s, &sc, sbp);
                    nstm_out[count] = fs_index(&s, &nc, bp_from_hand(nstm, owner, slot, i));
                    count++;
                }
            }
        }
    return count;
}

/* ---- synthetic PackedSfenValue records --------------------------------------------------------------------------
 * The reference has no encoder and no generator (its benchmark data is a private teacher file).  The benchmark's
 * stand-in is a seeded generator whose draw order is part of its definition; it is restated here so that the CPU arm
 * of the benchmark and the tests can produce the very same records without the CUDA library.  The bit stream is the
 * inverse of the decoder above (packed_sfen.rs:387-448).
 * Per record, from one SplitMix64 stream: side to move (low bit of a draw), black king square (uniform of 81), white
 * king square (uniform of the other 80); then each of the 38 other pieces in the order 18 pawns, 4 lances, 4 knights,
 * 4 silvers, 4 golds, 2 bishops, 2 rooks: on the board with p = 0.85 (uniform empty square in square order, uniform
 * owner, promoted with p = 0.1 unless gold), else in the hand of a uniform side; score = round-to-even(400 * N(0,1))
 * by Box-Muller, clipped to +-3000; result: draw with p = 0.05, else win with p = sigmoid(score / 600), else loss;
 * ply uniform in 1..256. */
typedef struct { uint64_t s; } sm64;
static uint64_t sm64_next(sm64* r) {
    uint64_t z = (r->s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static double sm64_unit(sm64* r) { return (double)(sm64_next(r) >> 11) * (1.0 / 9007199254740992.0); }
static uint32_t sm64_below(sm64* r, uint32_t n) { return (uint32_t)(((sm64_next(r) >> 32) * (uint64_t)n) >> 32); }

static void put_bits(uint8_t* data, int* cur, uint32_t v, int n) {
    for (int i = 0; i < n; ++i, ++*cur)
        if ((v >> i) & 1u) data[*cur >> 3] |= (uint8_t)(1u << (*cur & 7));
}
static int huff_id_for(uint8_t base_pt) {
    for (int id = 1; id < 8; ++id)
        if (HUFF_PT[id] == base_pt) return id;
    return 0;
}
static uint8_t unpromote_pt(uint8_t pt, int* promoted) {
    static const uint8_t base_of[6] = {PT_PAWN, PT_LANCE, PT_KNIGHT, PT_SILVER, PT_BISHOP, PT_ROOK};
    static const uint8_t pro_of[6] = {PT_PRO_PAWN, PT_PRO_LANCE, PT_PRO_KNIGHT, PT_PRO_SILVER, PT_HORSE, PT_DRAGON};
    *promoted = 0;
    for (int i = 0; i < 6; ++i)
        if (pt == pro_of[i]) { *promoted = 1; return base_of[i]; }
    return pt;
}

int ora_psv_encode(const ora_board* b, uint8_t* out) {
    memset(out, 0, 40);
    int cur = 0;
    put_bits(out, &cur, b->side_to_move & 1u, 1);
    put_bits(out, &cur, b->black_king_sq, 7);
    put_bits(out, &cur, b->white_king_sq, 7);
    for (int sq = 0; sq < 81; ++sq) {
        if (sq == b->black_king_sq || sq == b->white_king_sq) continue;
        if (b->board_pt[sq] == PT_NONE) { put_bits(out, &cur, 0, 1); continue; }
        int promoted;
        int id = huff_id_for(unpromote_pt(b->board_pt[sq], &promoted));
        if (id == 0) return -1;
        put_bits(out, &cur, HUFF_PATTERN[id], HUFF_BITS[id]);
        if (id != HUFF_GOLD) put_bits(out, &cur, (uint32_t)promoted, 1);
        put_bits(out, &cur, b->board_color[sq] & 1u, 1);
        if (cur > 256) return -1;
    }
    static const uint8_t slot_pt[7] = {PT_PAWN, PT_LANCE, PT_KNIGHT, PT_SILVER, PT_GOLD, PT_BISHOP, PT_ROOK};
    for (int color = 0; color < 2; ++color)
        for (int slot = 0; slot < 7; ++slot)
            for (int k = 0; k < b->hand[color][slot]; ++k) {
                int id = huff_id_for(slot_pt[slot]);
                put_bits(out, &cur, (uint32_t)HUFF_PATTERN[id] >> 1, HUFF_BITS[id] - 1);
                if (id != HUFF_GOLD) put_bits(out, &cur, 0, 1); /* piece-box flag */
                put_bits(out, &cur, (uint32_t)color, 1);
                if (cur > 256) return -1;
            }
    out[32] = (uint8_t)(b->score & 0xff);
    out[33] = (uint8_t)(((uint16_t)b->score >> 8) & 0xff);
    out[36] = (uint8_t)(b->ply & 0xff);
    out[37] = (uint8_t)((b->ply >> 8) & 0xff);
    out[38] = (uint8_t)b->result;
    return 0;
}

int ora_psv_synthesize(uint64_t seed, size_t n_records, uint8_t* out) {
    static const uint8_t kinds[7] = {PT_PAWN, PT_LANCE, PT_KNIGHT, PT_SILVER, PT_GOLD, PT_BISHOP, PT_ROOK};
    static const int copies[7] = {18, 4, 4, 4, 4, 2, 2};
    sm64 rng = {seed};
    for (size_t r = 0; r < n_records; ++r) {
        ora_board b;
        memset(&b, 0, sizeof b);
        b.side_to_move = (uint8_t)(sm64_next(&rng) & 1u);
        b.black_king_sq = (uint8_t)sm64_below(&rng, 81);
        int wk = (int)sm64_below(&rng, 80);
        if (wk >= b.black_king_sq) ++wk;
        b.white_king_sq = (uint8_t)wk;
        b.board_pt[b.black_king_sq] = PT_KING; b.board_color[b.black_king_sq] = 0;
        b.board_pt[wk] = PT_KING; b.board_color[wk] = 1;
        int empties = 79;
        for (int t = 0; t < 7; ++t)
            for (int k = 0; k < copies[t]; ++k) {
                if (sm64_unit(&rng) < 0.85) {
                    int pick = (int)sm64_below(&rng, (uint32_t)empties), sq = 0;
                    for (;; ++sq)
                        if (b.board_pt[sq] == PT_NONE && pick-- == 0) break;
                    int owner = (int)(sm64_next(&rng) & 1u);
                    uint8_t placed = kinds[t];
                    if (kinds[t] != PT_GOLD && sm64_unit(&rng) < 0.1) placed = promote_pt(kinds[t]);
                    b.board_pt[sq] = placed;
                    b.board_color[sq] = (uint8_t)owner;
                    --empties;
                } else {
                    int owner = (int)(sm64_next(&rng) & 1u);
                    b.hand[owner][hand_slot(kinds[t])]++;
                }
            }
        double u1 = sm64_unit(&rng);
        if (u1 < 1e-300) u1 = 1e-300;
        double u2 = sm64_unit(&rng);
        double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
        long sc = lrint(z * 400.0);
        if (sc > 3000) sc = 3000;
        if (sc < -3000) sc = -3000;
        b.score = (int16_t)sc;
        if (sm64_unit(&rng) < 0.05) b.result = 0;
        else b.result = sm64_unit(&rng) < 1.0 / (1.0 + exp(-(double)sc / 600.0)) ? 1 : -1;
        b.ply = (uint16_t)(1 + sm64_below(&rng, 256));
        if (ora_psv_encode(&b, out + 40 * r)) return -1;
    }
    return 0;
}

/* crates/shogi-features/src/kingrank9.rs:11-24 */
int ora_kingrank9_bucket(const ora_board* b) {
    int friendly, enemy;
    if (b->side_to_move == 0) { friendly = b->black_king_sq; enemy = 80 - b->white_king_sq; }
    else { friendly = 80 - b->white_king_sq; enemy = b->black_king_sq; }
    return ((friendly % 9) / 3) * 3 + (enemy % 9) / 3;
}

/* crates/nnue-train/src/dataloader.rs:444-500 (Batch::push_decoded_counting) + :322 (bucket) */
int ora_psv_to_batch(int feature_set, const uint8_t* psv, size_t n_records, int32_t* stm_idx,
                     int32_t* nstm_idx, int32_t* nnz, int32_t* bucket, float* score, float* wdl) {
    fs_spec s;
    if (fs_get(feature_set, &s)) return -1;
    int A = s.max_active;
    int err = 0;
    PAR_FOR
    for (size_t i = 0; i < n_records; ++i) {
        ora_board b;
        ora_psv_decode(psv + 40 * i, &b);
        for (int a = 0; a < A; ++a) { stm_idx[i * A + a] = -1; nstm_idx[i * A + a] = -1; }
        int n = ora_extract_active_features(feature_set, &b, stm_idx + i * A, nstm_idx + i * A, A);
        if (n > A) err = 1;
        nnz[i] = n;
        score[i] = (float)b.score;
        wdl[i] = b.result > 0 ? 1.0f : (b.result < 0 ? 0.0f : 0.5f);
        if (bucket) bucket[i] = ora_kingrank9_bucket(&b);
    }
    return err ? -2 : 0;
}

/* bins/nnue_train/src/loader_digest.rs:64-84 — the bytes fed to SHA-256 for one position */
size_t ora_loader_digest_bytes(const int32_t* stm, const int32_t* nstm, int32_t nnz, float score,
                               float wdl, uint8_t* out) {
    size_t o = 0;
    memcpy(out + o, &score, 4); o += 4;
    memcpy(out + o, &wdl, 4); o += 4;
    memcpy(out + o, &nnz, 4); o += 4;
    memcpy(out + o, stm, 4 * (size_t)nnz); o += 4 * (size_t)nnz;
    memcpy(out + o, nstm, 4 * (size_t)nnz); o += 4 * (size_t)nnz;
    return o;
}

/* ================================================================================
 * whole-step trainers
 * ================================================================================ */
#define MAX_GROUPS 10
#define FT_POST_SCALE (127.0f / 128.0f) /* bins/nnue_train/src/arch.rs:64-70 */
#define L1_SQR_SCALE (127.0f / 128.0f)
#define CLAMP_Q (127.0f / 64.0f) /* arch.rs:138-143: i8::MAX / QB */
#define CLAMP_NONE 3.402823466e+38f
#define BETA2 0.999f
#define EPS 1e-8f
#define RANGER_ALPHA 0.5f
#define RANGER_K 6
#define N_SMA_THRESHOLD 5.0f

typedef struct {
    const char* name;
    int kind; /* 0 ft, 1 dense, 2 bias */
    float clamp;
    size_t len;
    float *w, *m, *v, *slow, *grad;
} group;

struct ora_trainer {
    ora_config cfg;
    int cap;
    int n_groups;
    group g[MAX_GROUPS];
    uint64_t step_count;
    float* comb; /* folded forward table [N, F] (NULL without factorizer) */
    /* workspace */
    float *ft_stm, *ft_nstm, *combined, *dcombined, *dcombined2, *dft_stm, *dft_nstm;
    float *l1_bucket, *l1_shared, *l1_total, *l1_main, *l1_skip, *l1_sqr, *l2_pre, *l2_input, *l2_dense, *l2_acted;
    float *l3_out, *net_output, *dy, *norm;
    float *dl2_acted, *dl2_out, *dl2_input, *dl2_pre, *dl1_sqr, *dl1_mc, *dl1_ms, *dl1_main, *dl1_total;
    /* simple */
    float *l1_pre, *l1_acted, *dl1_acted, *dl1_pre;
    int32_t* idx_tmp;
    int last_n;
    /* reduced precision: bit 1 tf32, 2 ft_fp16, 4 ft_fp16_out, 8 fp16_opt_state (cli.rs:623-638) */
    int precision;
    float *table_h, *gtmp, *x_t, *w_t, *ws_t, *dl1_t; /* fp16 forward table; FT gradient of one perspective; tf32 operands */
    uint64_t clamp_count, clamp_elems;
};

static float* falloc(size_t n) { return (float*)calloc(n ? n : 1, sizeof(float)); }

static void add_group(ora_trainer* t, const char* name, int kind, float clamp, size_t len) {
    group* g = &t->g[t->n_groups++];
    g->name = name; g->kind = kind; g->clamp = clamp; g->len = len;
    g->w = falloc(len); g->m = falloc(len); g->v = falloc(len); g->slow = falloc(len); g->grad = falloc(len);
}

/* group tables: trainer_layerstack.rs:740-762 (+ft_w first), trainer_simple.rs:2497-2578 */
ora_trainer* ora_trainer_create(const ora_config* cfg, int cap) {
    ora_trainer* t = (ora_trainer*)calloc(1, sizeof(*t));
    t->cfg = *cfg;
    t->cap = cap;
    size_t N = (size_t)cfg->ft_in, F = (size_t)cfg->ft_out, l1 = (size_t)cfg->l1, l2 = (size_t)cfg->l2;
    size_t Nt = N + (cfg->factorize ? (size_t)cfg->piece_inputs : 0);
    size_t B = (size_t)cap;
    if (cfg->arch == 0) {
        size_t nb = (size_t)cfg->num_buckets, l1e = l1 - 1, l2in = 2 * l1e;
        add_group(t, "ft_w", 0, CLAMP_NONE, Nt * F);
        add_group(t, "ft_b", 2, CLAMP_NONE, F);
        add_group(t, "l1_w", 1, CLAMP_Q, nb * l1 * F);
        add_group(t, "l1_b", 2, CLAMP_Q, nb * l1);
        add_group(t, "l1_shared_weight", 1, CLAMP_Q, F * l1);
        add_group(t, "l1_shared_bias", 2, CLAMP_Q, l1);
        add_group(t, "l2_w", 1, CLAMP_Q, nb * l2 * l2in);
        add_group(t, "l2_b", 2, CLAMP_Q, nb * l2);
        add_group(t, "l3_w", 1, CLAMP_Q, nb * l2);
        add_group(t, "l3_b", 2, CLAMP_NONE, nb);
        t->combined = falloc(B * F); t->dcombined = falloc(B * F); t->dcombined2 = falloc(B * F);
        t->l1_bucket = falloc(B * l1); t->l1_shared = falloc(B * l1); t->l1_total = falloc(B * l1);
        t->l1_main = falloc(B * l1e); t->l1_skip = falloc(B); t->l1_sqr = falloc(B * l1e);
        t->l2_pre = falloc(B * l2in); t->l2_input = falloc(B * l2in); t->l2_dense = falloc(B * l2);
        t->l2_acted = falloc(B * l2); t->l3_out = falloc(B);
        t->dl2_acted = falloc(B * l2); t->dl2_out = falloc(B * l2); t->dl2_input = falloc(B * l2in);
        t->dl2_pre = falloc(B * l2in); t->dl1_sqr = falloc(B * l1e); t->dl1_mc = falloc(B * l1e);
        t->dl1_ms = falloc(B * l1e); t->dl1_main = falloc(B * l1e); t->dl1_total = falloc(B * l1);
    } else {
        add_group(t, "ft_w", 0, CLAMP_NONE, Nt * F);
        add_group(t, "ft_b", 2, CLAMP_NONE, F);
        add_group(t, "l1_w", 1, CLAMP_Q, (cfg->activation == 2 ? F : 2 * F) * l1); /* Pairwise: the L1 input is ft_out wide */
        add_group(t, "l1_b", 2, CLAMP_Q, l1);
        add_group(t, "l2_w", 1, CLAMP_Q, l1 * l2);
        add_group(t, "l2_b", 2, CLAMP_Q, l2);
        add_group(t, "l3_w", 1, CLAMP_Q, l2);
        add_group(t, "l3_b", 2, CLAMP_NONE, 1);
        t->combined = falloc(B * 2 * F); t->dcombined = falloc(B * 2 * F);
        t->l1_pre = falloc(B * l1); t->l1_acted = falloc(B * l1); t->l2_pre = falloc(B * l2); t->l2_acted = falloc(B * l2);
        t->dl2_acted = falloc(B * l2); t->dl2_pre = falloc(B * l2); t->dl1_acted = falloc(B * l1); t->dl1_pre = falloc(B * l1);
    }
    t->ft_stm = falloc(B * F); t->ft_nstm = falloc(B * F); t->dft_stm = falloc(B * F); t->dft_nstm = falloc(B * F);
    t->net_output = falloc(B); t->dy = falloc(B); t->norm = falloc(B);
    t->idx_tmp = (int32_t*)calloc(B * (size_t)cfg->max_active + 1, sizeof(int32_t));
    if (cfg->factorize) t->comb = falloc(N * F);
    return t;
}

void ora_trainer_destroy(ora_trainer* t) {
    if (!t) return;
    for (int i = 0; i < t->n_groups; ++i) { free(t->g[i].w); free(t->g[i].m); free(t->g[i].v); free(t->g[i].slow); free(t->g[i].grad); }
    float* bufs[] = {t->comb, t->ft_stm, t->ft_nstm, t->combined, t->dcombined, t->dcombined2, t->dft_stm, t->dft_nstm,
                     t->l1_bucket, t->l1_shared, t->l1_total, t->l1_main, t->l1_skip, t->l1_sqr, t->l2_pre, t->l2_input,
                     t->l2_dense, t->l2_acted, t->l3_out, t->net_output, t->dy, t->norm, t->dl2_acted, t->dl2_out,
                     t->dl2_input, t->dl2_pre, t->dl1_sqr, t->dl1_mc, t->dl1_ms, t->dl1_main, t->dl1_total,
                     t->l1_pre, t->l1_acted, t->dl1_acted, t->dl1_pre};
    for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); ++i) free(bufs[i]);
    free(t->idx_tmp);
    free(t->table_h); free(t->gtmp); free(t->x_t); free(t->w_t); free(t->ws_t); free(t->dl1_t);
    free(t);
}

void ora_trainer_set_precision(ora_trainer* t, int flags) { t->precision = flags; }
void ora_trainer_clamp_count(const ora_trainer* t, uint64_t* clamps, uint64_t* elems) {
    if (clamps) *clamps = t->clamp_count;
    if (elems) *elems = t->clamp_elems;
}
int ora_trainer_num_groups(const ora_trainer* t) { return t->n_groups; }
const char* ora_trainer_group_name(const ora_trainer* t, int g) { return t->g[g].name; }
size_t ora_trainer_group_len(const ora_trainer* t, int g) { return t->g[g].len; }
float* ora_trainer_group_ptr(ora_trainer* t, int gi, int which) {
    group* g = &t->g[gi];
    switch (which) { case 0: return g->w; case 1: return g->m; case 2: return g->v; case 3: return g->slow; case 4: return g->grad; }
    return NULL;
}
uint64_t ora_trainer_step_count(const ora_trainer* t) { return t->step_count; }
void ora_trainer_set_step_count(ora_trainer* t, uint64_t s) { t->step_count = s; }
void ora_trainer_set_threads(ora_trainer* t, int n) { (void)t; g_threads = n < 1 ? 1 : n; }

/* init.rs:213-316 (default_uniform) with the call shapes of trainer_layerstack.rs:844-878 and
 * trainer_simple.rs:454-463: real FT rows sampled at base shape, virtual rows appended as zeros. */
void ora_trainer_init_default(ora_trainer* t) {
    const ora_config* c = &t->cfg;
    size_t N = (size_t)c->ft_in, F = (size_t)c->ft_out;
    for (int i = 0; i < t->n_groups; ++i) {
        memset(t->g[i].w, 0, t->g[i].len * sizeof(float));
        memset(t->g[i].m, 0, t->g[i].len * sizeof(float));
        memset(t->g[i].v, 0, t->g[i].len * sizeof(float));
        memset(t->g[i].slow, 0, t->g[i].len * sizeof(float));
        memset(t->g[i].grad, 0, t->g[i].len * sizeof(float));
    }
    if (c->arch == 0) {
        size_t nb = (size_t)c->num_buckets, l1 = (size_t)c->l1, l2 = (size_t)c->l2, l2in = 2 * (l1 - 1);
        ora_init_sample(t->g[0].w, N * F, 1, N, 1, 1, 1.0f, 0, 0x100);
        ora_init_sample(t->g[2].w, nb * l1 * F, nb, F, 1, 0, 0.01f, 0, 0x101);
        ora_init_sample(t->g[4].w, F * l1, 1, F, 1, 0, 0.01f, 0, 0x102);
        ora_init_sample(t->g[6].w, nb * l2 * l2in, nb, l2in, 1, 0, 0.01f, 0, 0x103);
        ora_init_sample(t->g[8].w, nb * l2, nb, l2, 1, 0, 0.01f, 0, 0x104);
    } else {
        size_t l1 = (size_t)c->l1, l2 = (size_t)c->l2;
        ora_init_sample(t->g[0].w, N * F, 1, N, 1, 0, 0.01f, 0, 0x5071e001ull);
        ora_init_sample(t->g[1].w, F, 1, N, 1, 0, 0.01f, 0, 0x5071e002ull);
        ora_init_sample(t->g[2].w, 2 * F * l1, 1, 2 * F, 1, 0, 0.01f, 0, 0x5071e003ull);
        ora_init_sample(t->g[3].w, l1, 1, 2 * F, 1, 0, 0.01f, 0, 0x5071e004ull);
        ora_init_sample(t->g[4].w, l1 * l2, 1, l1, 1, 0, 0.01f, 0, 0x5071e005ull);
        ora_init_sample(t->g[5].w, l2, 1, l1, 1, 0, 0.01f, 0, 0x5071e006ull);
        ora_init_sample(t->g[6].w, l2, 1, l2, 1, 0, 0.01f, 0, 0x5071e007ull);
        ora_init_sample(t->g[7].w, 1, 1, l2, 1, 0, 0.01f, 0, 0x5071e008ull);
    }
}

const float* ora_trainer_buffer(const ora_trainer* t, const char* name, size_t* len) {
    const ora_config* c = &t->cfg;
    size_t B = (size_t)t->last_n, F = (size_t)c->ft_out;
    struct { const char* n; const float* p; size_t l; } tab[] = {
        {"ft_stm", t->ft_stm, B * F}, {"ft_nstm", t->ft_nstm, B * F},
        {"combined", t->combined, B * F * ((c->arch == 0 || c->activation == 2) ? 1 : 2)},
        {"l1_total", c->arch == 0 ? t->l1_total : t->l1_pre, B * (size_t)c->l1},
        {"net_output", t->net_output, B}, {"dy", t->dy, B},
        {"dl1_total", c->arch == 0 ? t->dl1_total : t->dl1_pre, B * (size_t)c->l1},
        {"dcombined", t->dcombined, B * F * ((c->arch == 0 || c->activation == 2) ? 1 : 2)},
        {"dft_stm", t->dft_stm, B * F}, {"dft_nstm", t->dft_nstm, B * F},
        {"comb", t->comb, t->comb ? (size_t)c->ft_in * F : 0},
    };
    for (size_t i = 0; i < sizeof(tab) / sizeof(tab[0]); ++i)
        if (strcmp(tab[i].n, name) == 0) { if (len) *len = tab[i].l; return tab[i].p; }
    return NULL;
}

static const float* forward_table(ora_trainer* t) {
    const ora_config* c = &t->cfg;
    size_t NF = (size_t)c->ft_in * (size_t)c->ft_out;
    const float* table = t->g[0].w;
    if (c->factorize) {
        /* the reference keeps comb in sync after every optimizer step / upload (trainer_layerstack.rs
         * launch_ft_fold); recomputing it from the current master weights here is the same thing. */
        ora_ft_fold_virtual(t->g[0].w, t->comb, (size_t)c->ft_in, (size_t)c->ft_out, (size_t)c->piece_inputs);
        table = t->comb;
    }
    if (t->precision & 2) {
        /* --ft-fp16: the forward reads an fp16 table: ft_fold_virtual_f16 (native_kernels.cu:262-318) with the factorizer,
         * else the mirror the optimizer kernels write (radam_step_*_mirror, ranger_lookahead_lerp_fp16_mirror) */
        if (!t->table_h) t->table_h = falloc(NF);
        PAR_FOR
        for (size_t i = 0; i < NF; ++i) t->table_h[i] = ora_round_half(table[i]);
        table = t->table_h;
    }
    return table;
}

static double run_loss(ora_trainer* t, const float* score, const float* wdl, int n, float lambda, const ora_loss* L) {
    double acc = 0.0;
    if (L->kind == 0)
        ora_loss_wdl(t->net_output, score, wdl, t->norm, t->dy, &acc, lambda, L->scale, (size_t)n);
    else {
        int extended = !(L->pow_exp == 2.0f && L->qp_asymmetry == 0.0f && L->weight_boost_w1 == 0.0f);
        ora_loss_wrm(t->net_output, score, wdl, t->norm, t->dy, &acc, lambda, L->nnue2score, L->in_scaling,
                     L->in_offset, L->target_offset, L->target_scaling, L->pow_exp, L->qp_asymmetry,
                     L->weight_boost_w1, L->weight_boost_w2, extended, (size_t)n);
    }
    return acc;
}

/* forward of trainer_layerstack.rs:2038-2848 (fp32, no psqt) */
static double ls_forward(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                         const int32_t* bucket, const float* score, const float* wdl, int n, float lambda,
                         const ora_loss* L) {
    const ora_config* c = &t->cfg;
    size_t B = (size_t)n, F = (size_t)c->ft_out, N = (size_t)c->ft_in, A = (size_t)c->max_active;
    size_t l1 = (size_t)c->l1, l2 = (size_t)c->l2, nb = (size_t)c->num_buckets, l1e = l1 - 1, l2in = 2 * l1e;
    const float* table = forward_table(t);
    ora_sparse_ft_forward(table, stm_idx, nnz, t->ft_stm, B, F, N, A);   /* fp16 rows are summed in fp32 (:743-801) */
    ora_sparse_ft_forward(table, nstm_idx, nnz, t->ft_nstm, B, F, N, A);
    if (t->precision & 4) { /* sparse_ft_forward_fp16_out: the sums are stored as fp16; ft_post_perspective_fwd_fp16 reads them */
        PAR_FOR
        for (size_t i = 0; i < B * F; ++i) { t->ft_stm[i] = ora_round_half(t->ft_stm[i]); t->ft_nstm[i] = ora_round_half(t->ft_nstm[i]); }
    }
    ora_ft_post_perspective_fwd(t->ft_stm, t->ft_nstm, t->g[1].w, t->combined, B, F, FT_POST_SCALE);
    const float *x1 = t->combined, *w1 = t->g[2].w, *ws1 = t->g[4].w;
    if (t->precision & 1) { /* --tf32: every L1 product runs on TF32 operands (trainer_layerstack.rs:2388-2420, 2498-2506) */
        if (!t->x_t) { t->x_t = falloc((size_t)t->cap * F); t->w_t = falloc(nb * l1 * F); t->ws_t = falloc(F * l1); t->dl1_t = falloc((size_t)t->cap * l1); }
        PAR_FOR
        for (size_t i = 0; i < B * F; ++i) t->x_t[i] = ora_tf32(t->combined[i]);
        for (size_t i = 0; i < nb * l1 * F; ++i) t->w_t[i] = ora_tf32(t->g[2].w[i]);
        for (size_t i = 0; i < F * l1; ++i) t->ws_t[i] = ora_tf32(t->g[4].w[i]);
        x1 = t->x_t; w1 = t->w_t; ws1 = t->ws_t;
    }
    ora_dense_mm_fwd_bucket(x1, w1, t->g[3].w, bucket, t->l1_bucket, B, F, l1, nb);
    ora_dense_mm_fwd(x1, ws1, t->g[5].w, t->l1_shared, B, F, l1);
    ora_elementwise_add(t->l1_bucket, t->l1_shared, t->l1_total, B * l1);
    ora_slice_extract_2d(t->l1_total, t->l1_main, B, l1, 0, l1e);
    ora_slice_extract_2d(t->l1_total, t->l1_skip, B, l1, l1e, 1);
    ora_abs_pow2_scale_fwd(t->l1_main, t->l1_sqr, L1_SQR_SCALE, B * l1e);
    ora_concat_l1sqr_main_fwd(t->l1_sqr, t->l1_main, t->l2_pre, B, l1e, l1e);
    ora_crelu_fwd(t->l2_pre, t->l2_input, B * l2in);
    ora_dense_mm_fwd_bucket(t->l2_input, t->g[6].w, t->g[7].w, bucket, t->l2_dense, B, l2in, l2, nb);
    ora_crelu_fwd(t->l2_dense, t->l2_acted, B * l2);
    ora_dense_mm_fwd_bucket(t->l2_acted, t->g[8].w, t->g[9].w, bucket, t->l3_out, B, l2, 1, nb);
    ora_elementwise_add(t->l3_out, t->l1_skip, t->net_output, B);
    return run_loss(t, score, wdl, n, lambda, L);
}

/* the GPU path limits the FT backward to the first nnz slots (native_kernels.cu build_feature_counts),
 * the CPU function scans every slot: mask the tail so both agree. */
static const int32_t* masked_indices(ora_trainer* t, const int32_t* idx, const int32_t* nnz, size_t B, size_t A) {
    for (size_t b = 0; b < B; ++b)
        for (size_t a = 0; a < A; ++a) t->idx_tmp[b * A + a] = (int32_t)a < nnz[b] ? idx[b * A + a] : -1;
    return t->idx_tmp;
}

static void zero_grads(ora_trainer* t) {
    for (int i = 0; i < t->n_groups; ++i) memset(t->g[i].grad, 0, t->g[i].len * sizeof(float));
}

static void ft_backward(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz, size_t B) {
    const ora_config* c = &t->cfg;
    size_t F = (size_t)c->ft_out, N = (size_t)c->ft_in, A = (size_t)c->max_active;
    ora_sparse_ft_backward(t->dft_stm, masked_indices(t, stm_idx, nnz, B, A), t->g[0].grad, B, F, N, A);
    ora_sparse_ft_backward(t->dft_nstm, masked_indices(t, nstm_idx, nnz, B, A), t->g[0].grad, B, F, N, A);
    if (c->factorize) ora_ft_reduce_virtual_grad(t->g[0].grad, N, F, (size_t)c->piece_inputs);
}

/* --ft-fp16-out: ft_post_perspective_grad_fused_fp16 (native_kernels.cu:2304-2353) stores dft * gradient_scale clamped to
 * the fp16 range (clamps counted) and rounded, with gradient_scale = 2^14 * batch (trainer_layerstack.rs:3617-3621, the
 * bias gradient takes the unscaled value); gather_and_sum_per_feature_{overwrite,add}_fp16 (:1081-1181) sum the fp16 rows
 * of one perspective in fp32, multiply by 1 / gradient_scale, and the second perspective is added to the first. */
static void ft_backward_fp16(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz, size_t B) {
    const ora_config* c = &t->cfg;
    size_t F = (size_t)c->ft_out, N = (size_t)c->ft_in, A = (size_t)c->max_active;
    size_t Nt = N + (c->factorize ? (size_t)c->piece_inputs : 0);
    float scale = 16384.0f * (float)B, inv = 1.0f / scale;
    if (!t->gtmp) t->gtmp = falloc(Nt * F);
    uint64_t clamps = 0;
    for (int p = 0; p < 2; ++p) {
        float* d = p == 0 ? t->dft_stm : t->dft_nstm;
        for (size_t i = 0; i < B * F; ++i) d[i] = ora_round_half(clamp_half_count(d[i] * scale, &clamps)); /* the stored fp16 rows */
        memset(t->gtmp, 0, N * F * sizeof(float));
        ora_sparse_ft_backward(d, masked_indices(t, p == 0 ? stm_idx : nstm_idx, nnz, B, A), t->gtmp, B, F, N, A);
        float* g = t->g[0].grad;
        PAR_FOR
        for (size_t i = 0; i < N * F; ++i) g[i] = p == 0 ? t->gtmp[i] * inv : g[i] + t->gtmp[i] * inv;
        PAR_FOR
        for (size_t i = 0; i < B * F; ++i) d[i] *= inv; /* reported in the gradient's own scale */
    }
    t->clamp_count += clamps;
    t->clamp_elems += 2 * (uint64_t)B * (uint64_t)F;
    if (c->factorize) ora_ft_reduce_virtual_grad(t->g[0].grad, N, F, (size_t)c->piece_inputs);
}

/* backward of trainer_layerstack.rs:2849-4032 */
static void ls_backward(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                        const int32_t* bucket, int n) {
    const ora_config* c = &t->cfg;
    size_t B = (size_t)n, F = (size_t)c->ft_out;
    size_t l1 = (size_t)c->l1, l2 = (size_t)c->l2, nb = (size_t)c->num_buckets, l1e = l1 - 1, l2in = 2 * l1e;
    zero_grads(t);
    ora_dense_mm_bwd_input_bucket(t->dy, t->g[8].w, bucket, t->dl2_acted, B, l2, 1, nb);
    ora_dense_mm_bwd_weight_bucket(t->l2_acted, t->dy, bucket, t->g[8].grad, B, l2, 1, nb);
    ora_bias_grad_bucket(t->dy, bucket, t->g[9].grad, B, 1, nb);
    ora_crelu_grad(t->l2_dense, t->dl2_acted, t->dl2_out, B * l2);
    ora_dense_mm_bwd_input_bucket(t->dl2_out, t->g[6].w, bucket, t->dl2_input, B, l2in, l2, nb);
    ora_dense_mm_bwd_weight_bucket(t->l2_input, t->dl2_out, bucket, t->g[6].grad, B, l2in, l2, nb);
    ora_bias_grad_bucket(t->dl2_out, bucket, t->g[7].grad, B, l2, nb);
    ora_crelu_grad(t->l2_pre, t->dl2_input, t->dl2_pre, B * l2in);
    ora_concat_l1sqr_main_grad(t->dl2_pre, t->dl1_sqr, t->dl1_mc, B, l1e);
    ora_abs_pow2_scale_grad(t->l1_main, t->dl1_sqr, t->dl1_ms, L1_SQR_SCALE, B * l1e);
    ora_elementwise_add(t->dl1_mc, t->dl1_ms, t->dl1_main, B * l1e);
    memset(t->dl1_total, 0, B * l1 * sizeof(float));
    ora_slice_scatter_2d(t->dl1_main, t->dl1_total, B, l1e, l1, 0);
    ora_slice_scatter_2d(t->dy, t->dl1_total, B, 1, l1, l1e);
    const float *x1 = t->combined, *w1 = t->g[2].w, *ws1 = t->g[4].w, *d1 = t->dl1_total;
    if (t->precision & 1) { /* --tf32: the four L1 gradient products too (trainer_layerstack.rs:3340-3398, 3454-3541) */
        PAR_FOR
        for (size_t i = 0; i < B * l1; ++i) t->dl1_t[i] = ora_tf32(t->dl1_total[i]);
        x1 = t->x_t; w1 = t->w_t; ws1 = t->ws_t; d1 = t->dl1_t; /* operands of the forward are unchanged */
    }
    /* L1 shared */
    ora_dense_mm_bwd_input(d1, ws1, t->dcombined2, B, F, l1);
    ora_dense_mm_bwd_weight(x1, d1, t->g[4].grad, B, F, l1);
    ora_bias_grad(t->dl1_total, t->g[5].grad, B, l1);
    /* L1 per bucket */
    ora_dense_mm_bwd_weight_bucket(x1, d1, bucket, t->g[2].grad, B, F, l1, nb);
    ora_dense_mm_bwd_input_bucket(d1, w1, bucket, t->dcombined, B, F, l1, nb);
    ora_bias_grad_bucket(t->dl1_total, bucket, t->g[3].grad, B, l1, nb);
    /* native_kernels.cu:2260 ft_post_perspective_grad_fused adds the two sources in-register */
    ora_elementwise_add(t->dcombined, t->dcombined2, t->dcombined, B * F);
    ora_ft_post_perspective_grad(t->dcombined, t->ft_stm, t->g[1].w, t->dft_stm, t->g[1].grad, B, F, 0, F, FT_POST_SCALE);
    ora_ft_post_perspective_grad(t->dcombined, t->ft_nstm, t->g[1].w, t->dft_nstm, t->g[1].grad, B, F, F / 2, F, FT_POST_SCALE);
    if (t->precision & 4) ft_backward_fp16(t, stm_idx, nstm_idx, nnz, B);
    else ft_backward(t, stm_idx, nstm_idx, nnz, B);
}

static void act_fwd(int act, const float* x, float* y, size_t n) { if (act == 0) ora_crelu_fwd(x, y, n); else ora_screlu_fwd(x, y, n); }
static void act_grad(int act, const float* x, const float* dy, float* dx, size_t n) {
    if (act == 0) ora_crelu_grad(x, dy, dx, n); else ora_screlu_grad(x, dy, dx, n);
}

/* forward of trainer_simple.rs:857-1508 (fp32, crelu/screlu) */
static double simple_forward(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                             const float* score, const float* wdl, int n, float lambda, const ora_loss* L) {
    const ora_config* c = &t->cfg;
    size_t B = (size_t)n, F = (size_t)c->ft_out, N = (size_t)c->ft_in, A = (size_t)c->max_active;
    size_t l1 = (size_t)c->l1, l2 = (size_t)c->l2;
    const float* table = forward_table(t);
    ora_sparse_ft_forward(table, stm_idx, nnz, t->ft_stm, B, F, N, A);
    ora_sparse_ft_forward(table, nstm_idx, nnz, t->ft_nstm, B, F, N, A);
    const float* bias = t->g[1].w;
    size_t K1 = c->activation == 2 ? F : 2 * F;
    int act = c->activation == 1 ? 1 : 0; /* the dense layers: SCReLU, or CReLU (also under Pairwise, trainer_simple.rs:1304) */
    if (c->activation == 2) /* SimpleActivation::Pairwise: the LayerStack FT post, raw sums kept (trainer_simple.rs:1241-1262) */
        ora_ft_post_perspective_fwd(t->ft_stm, t->ft_nstm, bias, t->combined, B, F, FT_POST_SCALE);
    /* native_kernels.cu:1406-1450 simple_ft_post_fused_*: x = ft + bias stored back, act -> combined */
    for (int p = 0; p < 2 && c->activation != 2; ++p) {
        float* ft = p == 0 ? t->ft_stm : t->ft_nstm;
        size_t off = p == 0 ? 0 : F;
        PAR_FOR
        for (size_t b = 0; b < B; ++b)
            for (size_t col = 0; col < F; ++col) {
                float v = ft[b * F + col] + bias[col];
                ft[b * F + col] = v;
                float a = crelu01(v);
                t->combined[b * 2 * F + off + col] = c->activation == 0 ? a : a * a;
            }
    }
    ora_dense_mm_fwd(t->combined, t->g[2].w, t->g[3].w, t->l1_pre, B, K1, l1);
    act_fwd(act, t->l1_pre, t->l1_acted, B * l1);
    ora_dense_mm_fwd(t->l1_acted, t->g[4].w, t->g[5].w, t->l2_pre, B, l1, l2);
    act_fwd(act, t->l2_pre, t->l2_acted, B * l2);
    ora_dense_mm_fwd(t->l2_acted, t->g[6].w, t->g[7].w, t->net_output, B, l2, 1);
    return run_loss(t, score, wdl, n, lambda, L);
}

/* backward of trainer_simple.rs:1509-2357 */
static void simple_backward(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz, int n) {
    const ora_config* c = &t->cfg;
    size_t B = (size_t)n, F = (size_t)c->ft_out, l1 = (size_t)c->l1, l2 = (size_t)c->l2;
    size_t K1 = c->activation == 2 ? F : 2 * F;
    int act = c->activation == 1 ? 1 : 0;
    zero_grads(t);
    ora_dense_mm_bwd_input(t->dy, t->g[6].w, t->dl2_acted, B, l2, 1);
    ora_dense_mm_bwd_weight(t->l2_acted, t->dy, t->g[6].grad, B, l2, 1);
    ora_bias_grad(t->dy, t->g[7].grad, B, 1);
    act_grad(act, t->l2_pre, t->dl2_acted, t->dl2_pre, B * l2);
    ora_dense_mm_bwd_input(t->dl2_pre, t->g[4].w, t->dl1_acted, B, l1, l2);
    ora_dense_mm_bwd_weight(t->l1_acted, t->dl2_pre, t->g[4].grad, B, l1, l2);
    ora_bias_grad(t->dl2_pre, t->g[5].grad, B, l2);
    act_grad(act, t->l1_pre, t->dl1_acted, t->dl1_pre, B * l1);
    ora_dense_mm_bwd_input(t->dl1_pre, t->g[2].w, t->dcombined, B, K1, l1);
    ora_dense_mm_bwd_weight(t->combined, t->dl1_pre, t->g[2].grad, B, K1, l1);
    ora_bias_grad(t->dl1_pre, t->g[3].grad, B, l1);
    if (c->activation == 2) { /* Pairwise: ft_post_perspective_grad per perspective, which also adds the bias gradient (trainer_simple.rs:2008-2040) */
        ora_ft_post_perspective_grad(t->dcombined, t->ft_stm, t->g[1].w, t->dft_stm, t->g[1].grad, B, F, 0, F, FT_POST_SCALE);
        ora_ft_post_perspective_grad(t->dcombined, t->ft_nstm, t->g[1].w, t->dft_nstm, t->g[1].grad, B, F, F / 2, F, FT_POST_SCALE);
        ft_backward(t, stm_idx, nstm_idx, nnz, B);
        return;
    }
    /* native_kernels.cu:1452-1497 simple_bwd_ft_act_*_fused (x is the biased pre-activation) */
    for (int p = 0; p < 2; ++p) {
        const float* x = p == 0 ? t->ft_stm : t->ft_nstm;
        float* d = p == 0 ? t->dft_stm : t->dft_nstm;
        size_t off = p == 0 ? 0 : F;
        PAR_FOR
        for (size_t b = 0; b < B; ++b)
            for (size_t col = 0; col < F; ++col) {
                float xv = x[b * F + col];
                float up = t->dcombined[b * 2 * F + off + col];
                if (c->activation == 0) d[b * F + col] = (xv > 0.0f && xv < 1.0f) ? up : 0.0f;
                else { float a = crelu01(xv); d[b * F + col] = up * ((a > 0.0f && a < 1.0f) ? 2.0f * a : 0.0f); }
            }
    }
    /* native_kernels.cu:1572 simple_bias_grad_dual: sum over rows of (stm + nstm) */
    float* gb = t->g[1].grad;
    PAR_FOR
    for (size_t col = 0; col < F; ++col) {
        float s = 0.0f;
        for (size_t b = 0; b < B; ++b) s += t->dft_stm[b * F + col] + t->dft_nstm[b * F + col];
        gb[col] += s;
    }
    ft_backward(t, stm_idx, nstm_idx, nnz, B);
}

/* trainer_layerstack.rs:4034-4482, trainer_simple.rs:2359-2675 */
void ora_trainer_apply_optimizer(ora_trainer* t, float lr) {
    const ora_config* c = &t->cfg;
    t->step_count += 1;
    float step_size, beta1;
    int32_t denom;
    ora_optimizer_scalars(c->optimizer, t->step_count, BETA2, N_SMA_THRESHOLD, &step_size, &denom, &beta1);
    const float wd[3] = {c->wd_ft, c->wd_dense, c->wd_bias};
    const float lm[3] = {c->lr_mult_ft, c->lr_mult_dense, c->lr_mult_bias};
    for (int i = 0; i < t->n_groups; ++i) {
        group* g = &t->g[i];
        if (i == 0 && (t->precision & 8)) /* --fp16-opt-state: only the FT table's moments (trainer_layerstack.rs:4085-4117) */
            ora_radam_step_f16state(g->w, g->m, g->v, g->grad, lr * lm[g->kind], step_size, denom, wd[g->kind], beta1, BETA2,
                                    EPS, -g->clamp, g->clamp, 268435456.0f /* 2^28 */, 1099511627776.0f /* 2^40 */, g->len);
        else
            ora_radam_step(g->w, g->m, g->v, g->grad, lr * lm[g->kind], step_size, denom, wd[g->kind], beta1, BETA2,
                           EPS, -g->clamp, g->clamp, g->len);
    }
    if (c->optimizer == 0 && t->step_count % RANGER_K == 0)
        for (int i = 0; i < t->n_groups; ++i) ora_ranger_lookahead_lerp(t->g[i].w, t->g[i].slow, RANGER_ALPHA, t->g[i].len);
}

double ora_trainer_step(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                        const int32_t* bucket_idx, const float* score, const float* wdl, int n_pos,
                        float per_pos_norm, float lr, float wdl_lambda, const ora_loss* loss, int do_optimizer) {
    if (n_pos <= 0 || n_pos > t->cap) return 0.0;
    t->last_n = n_pos;
    for (int i = 0; i < n_pos; ++i) t->norm[i] = per_pos_norm;
    double l;
    if (t->cfg.arch == 0) {
        l = ls_forward(t, stm_idx, nstm_idx, nnz, bucket_idx, score, wdl, n_pos, wdl_lambda, loss);
        ls_backward(t, stm_idx, nstm_idx, nnz, bucket_idx, n_pos);
    } else {
        l = simple_forward(t, stm_idx, nstm_idx, nnz, score, wdl, n_pos, wdl_lambda, loss);
        simple_backward(t, stm_idx, nstm_idx, nnz, n_pos);
    }
    if (do_optimizer) ora_trainer_apply_optimizer(t, lr);
    return l;
}

double ora_trainer_validate(ora_trainer* t, const int32_t* stm_idx, const int32_t* nstm_idx, const int32_t* nnz,
                            const int32_t* bucket_idx, const float* score, const float* wdl, int n_pos,
                            float wdl_lambda, const ora_loss* loss, float* net_output) {
    if (n_pos <= 0 || n_pos > t->cap) return 0.0;
    t->last_n = n_pos;
    for (int i = 0; i < n_pos; ++i) t->norm[i] = 1.0f / (float)n_pos;
    double l = t->cfg.arch == 0
                   ? ls_forward(t, stm_idx, nstm_idx, nnz, bucket_idx, score, wdl, n_pos, wdl_lambda, loss)
                   : simple_forward(t, stm_idx, nstm_idx, nnz, score, wdl, n_pos, wdl_lambda, loss);
    if (net_output) memcpy(net_output, t->net_output, (size_t)n_pos * sizeof(float));
    return l;
}

void ora_trainer_accumulate_grads(ora_trainer* dst, const ora_trainer* src) {
    for (int i = 0; i < dst->n_groups; ++i) {
        size_t n = dst->g[i].len;
        float* d = dst->g[i].grad;
        const float* s = src->g[i].grad;
        PAR_FOR
        for (size_t k = 0; k < n; ++k) d[k] += s[k];
    }
}
