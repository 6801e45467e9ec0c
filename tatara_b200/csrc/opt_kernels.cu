// Optimizer kernels: the RAdam / Ranger / AdamW update with weight clamp (radam_step,
// native_kernels.cu:1291; pointwise/radam_step.rs:116-156) and the Ranger look-ahead interpolation
// (native_kernels.cu:1842; pointwise/ranger_step.rs:52-59), fused so that every parameter and moment
// crosses HBM once per step.  The gradient is only read: every gradient buffer is fully rewritten by
// the next backward pass, so the reference's grad = 0 store is not needed.
#include "common.cuh"

#include <cuda_fp16.h>

static __device__ __forceinline__ unsigned ok_pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
}
static __device__ __forceinline__ float2 ok_unpack_h2(unsigned pair) { return __half22float2(*reinterpret_cast<const __half2*>(&pair)); }
static __device__ __forceinline__ uint2 pack_h4(float4 v) { return make_uint2(ok_pack_h2(v.x, v.y), ok_pack_h2(v.z, v.w)); }

// Four moments of one float4 of parameters.  fp32 state: as stored.  fp16 state (radam_step_f16state,
// native_kernels.cu:1127-1181): stored = clamp(value * scale) rounded to fp16; read back as stored / scale.  The update
// itself uses the unrounded new moments; the scales are powers of two, so scaling is exact.
template <bool HS>
static __device__ __forceinline__ float4 load_moment(const void* base, size_t i4, float inv_scale, bool streaming) {
    if (HS) {
        const uint2* p = static_cast<const uint2*>(base) + i4;
        const uint2 u = streaming ? __ldcs(p) : *p;
        const float2 a = ok_unpack_h2(u.x), b = ok_unpack_h2(u.y);
        return make_float4(a.x * inv_scale, a.y * inv_scale, b.x * inv_scale, b.y * inv_scale);
    }
    const float4* p = static_cast<const float4*>(base) + i4;
    return streaming ? __ldcs(p) : *p;
}
static __device__ __forceinline__ float clamp_h(float x, bool both) {
    x = x > 65504.0f ? 65504.0f : x;  // comparisons keep a NaN, as the reference does
    if (both) x = x < -65504.0f ? -65504.0f : x;
    return x;
}
template <bool HS>
static __device__ __forceinline__ void store_moment(void* base, size_t i4, float4 val, float scale, bool both, bool streaming) {
    if (HS) {
        const float4 q = make_float4(clamp_h(val.x * scale, both), clamp_h(val.y * scale, both), clamp_h(val.z * scale, both),
                                     clamp_h(val.w * scale, both));
        uint2* p = static_cast<uint2*>(base) + i4;
        if (streaming) __stcs(p, pack_h4(q)); else *p = pack_h4(q);
    } else {
        float4* p = static_cast<float4*>(base) + i4;
        if (streaming) __stcs(p, val); else *p = val;
    }
}
static __device__ __forceinline__ float4 scale4(float4 g, float k) { return make_float4(g.x * k, g.y * k, g.z * k, g.w * k); }

static __device__ __forceinline__ float radam_one(float p, float& m, float& v, float g, const OptScalars& sc, float rate,
                                                   float decay_mul) {
    p *= decay_mul;
    const float mi = sc.beta1 * m + (1.0f - sc.beta1) * g;
    const float vi = sc.beta2 * v + (1.0f - sc.beta2) * g * g;
    m = mi;
    v = vi;
    float val = mi;
    if (sc.denom != 0) val /= sqrtf(vi) + sc.eps;
    p -= rate * val;
    p = p < sc.min_w ? sc.min_w : p;
    p = p > sc.max_w ? sc.max_w : p;
    return p;
}

static __device__ __forceinline__ float4 radam_four(float4 p, float4& m, float4& v, float4 g, const OptScalars& sc,
                                                     float rate, float decay_mul) {
    float4 r;
    r.x = radam_one(p.x, m.x, v.x, g.x, sc, rate, decay_mul);
    r.y = radam_one(p.y, m.y, v.y, g.y, sc, rate, decay_mul);
    r.z = radam_one(p.z, m.z, v.z, g.z, sc, rate, decay_mul);
    r.w = radam_one(p.w, m.w, v.w, g.w, sc, rate, decay_mul);
    return r;
}

static __device__ __forceinline__ float4 lerp_four(float4 w, float4 s, float alpha) {
    const float oma = 1.0f - alpha;
    return make_float4(alpha * w.x + oma * s.x, alpha * w.y + oma * s.y, alpha * w.z + oma * s.z, alpha * w.w + oma * s.w);
}

// plain streaming update of one large group (n multiple of 4); mirror: optional fp16 copy of the updated weights
// (radam_step_fp16_mirror / radam_step_f16state_mirror + ranger_lookahead_lerp_fp16_mirror, native_kernels.cu:1183-1290)
template <bool HS>
__global__ void __launch_bounds__(256) k_radam(float4* __restrict__ w, void* __restrict__ m, void* __restrict__ v,
                                                const float4* __restrict__ g, float4* __restrict__ slow, uint2* __restrict__ mirror,
                                                long long n4, OptScalars sc) {
    const float rate = sc.lr * sc.step_size;
    const float decay_mul = 1.0f - sc.decay * rate;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        float4 mi = load_moment<HS>(m, i, 1.0f / TB_FT_OPT_M_SCALE, false), vi = load_moment<HS>(v, i, 1.0f / TB_FT_OPT_V_SCALE, false);
        float4 p = radam_four(w[i], mi, vi, scale4(g[i], sc.grad_scale), sc, rate, decay_mul);
        store_moment<HS>(m, i, mi, TB_FT_OPT_M_SCALE, true, false);
        store_moment<HS>(v, i, vi, TB_FT_OPT_V_SCALE, false, false);
        if (sc.lerp) {
            p = lerp_four(p, slow[i], sc.alpha);
            slow[i] = p;
        }
        w[i] = p;
        if (mirror) mirror[i] = pack_h4(p);
    }
}

int launch_radam(cudaStream_t s, float* w, void* m, void* v, const float* g, float* slow, int64_t n, OptScalars sc, int half_state,
                 void* mirror) {
    const long long n4 = n / 4;
    long long blocks = (n4 + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (blocks < 1) blocks = 1;
    if (half_state)
        k_radam<true><<<(int)blocks, 256, 0, s>>>(reinterpret_cast<float4*>(w), m, v, reinterpret_cast<const float4*>(g),
                                                  reinterpret_cast<float4*>(slow), static_cast<uint2*>(mirror), n4, sc);
    else
        k_radam<false><<<(int)blocks, 256, 0, s>>>(reinterpret_cast<float4*>(w), m, v, reinterpret_cast<const float4*>(g),
                                                   reinterpret_cast<float4*>(slow), static_cast<uint2*>(mirror), n4, sc);
    return 1;
}

// all small groups in one launch: grid (groups, blocks)
__global__ void __launch_bounds__(256) k_radam_small(const __grid_constant__ SmallGroups groups, OptScalars sc) {
    const SmallGroup gr = groups.g[blockIdx.x];
    sc.lr = gr.lr;
    sc.decay = gr.decay;
    sc.min_w = gr.min_w;
    sc.max_w = gr.max_w;
    const float rate = sc.lr * sc.step_size;
    const float decay_mul = 1.0f - sc.decay * rate;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < gr.n; i += gridDim.y * blockDim.x) {
        float mi = gr.m[i], vi = gr.v[i];
        float p = radam_one(gr.w[i], mi, vi, gr.grad[i], sc, rate, decay_mul);
        gr.m[i] = mi;
        gr.v[i] = vi;
        if (sc.lerp) {
            p = sc.alpha * p + (1.0f - sc.alpha) * gr.slow[i];
            gr.slow[i] = p;
        }
        gr.w[i] = p;
    }
}

int launch_radam_small(cudaStream_t s, const SmallGroups& groups, int max_n, OptScalars sc) {
    int by = ceil_div(max_n, 256 * 4);
    if (by < 1) by = 1;
    if (by > 512) by = 512;
    k_radam_small<<<dim3(groups.n, by), 256, 0, s>>>(groups, sc);
    return 1;
}

// ------------------------------------------------------------------------------------------------
// Factorised FT table (N = KB * pi real rows + pi virtual rows).  One block per virtual row v, one
// thread per float4 column:
//   pass 1: update the KB real rows kb*pi + v and add up their gradients in kb order
//           (ft_reduce_virtual_grad, sparse/ft_factorize.rs:109-121),
//   then update the virtual row N + v with that sum (and store the sum as its gradient),
//   pass 2: comb[kb*pi + v] = w[kb*pi + v] + w[N + v] (ft_fold_virtual, sparse/ft_factorize.rs:78-99);
//           the real rows were written a moment ago by this block and are read back from L2.
// Replaces radam_step on N_t*F elements + ft_reduce_virtual_grad + ranger_lookahead_lerp + ft_fold_virtual.
// Two builds: rows of up to 384 float4 (F <= 1536) run three blocks per SM (56 registers), longer rows one or two.
// ------------------------------------------------------------------------------------------------
// HS: fp16 moments; HC: fp16 folded table.  The real rows' gradients are multiplied by sc.grad_scale on load; the virtual
// row's gradient cell receives the sum of the scaled values (its true gradient).
template <int MAX_THREADS, int MIN_BLOCKS, bool HS, bool HC>
__global__ void __launch_bounds__(MAX_THREADS, MIN_BLOCKS) k_radam_factorized(float4* __restrict__ w, void* __restrict__ m, void* __restrict__ v,
                                                            float4* __restrict__ g, float4* __restrict__ slow,
                                                            void* __restrict__ comb, int N, int pi, int row4, OptScalars sc) {
    const float inv_ms = 1.0f / TB_FT_OPT_M_SCALE, inv_vs = 1.0f / TB_FT_OPT_V_SCALE;
    const int vr = blockIdx.x;
    const int c = threadIdx.x;
    const float rate = sc.lr * sc.step_size;
    const float decay_mul = 1.0f - sc.decay * rate;
    const int KB = N / pi;
    float4 gsum = make_float4(0.f, 0.f, 0.f, 0.f);
    // m, v and the gradient stream through once: evict-first loads / stores keep them from pushing the freshly
    // written weights out of L2 before pass 2 reads them back
#pragma unroll 4
    for (int kb = 0; kb < KB; ++kb) {
        const size_t i = (size_t)(kb * pi + vr) * row4 + c;
        float4 gi = __ldcs(g + i);
        if (HC) gi = scale4(gi, sc.grad_scale);  // loss-scaled sums exist only next to an fp16 table
        float4 mi = load_moment<HS>(m, i, inv_ms, true), vi = load_moment<HS>(v, i, inv_vs, true);
        float4 p = radam_four(w[i], mi, vi, gi, sc, rate, decay_mul);
        store_moment<HS>(m, i, mi, TB_FT_OPT_M_SCALE, true, true);
        store_moment<HS>(v, i, vi, TB_FT_OPT_V_SCALE, false, true);
        if (sc.lerp) {
            p = lerp_four(p, __ldcs(slow + i), sc.alpha);
            __stcs(slow + i, p);
        }
        w[i] = p;
        gsum.x += gi.x; gsum.y += gi.y; gsum.z += gi.z; gsum.w += gi.w;
    }
    const size_t iv = (size_t)(N + vr) * row4 + c;
    g[iv] = gsum;
    float4 mv = load_moment<HS>(m, iv, inv_ms, false), vv = load_moment<HS>(v, iv, inv_vs, false);
    float4 pv = radam_four(w[iv], mv, vv, gsum, sc, rate, decay_mul);
    store_moment<HS>(m, iv, mv, TB_FT_OPT_M_SCALE, true, false);
    store_moment<HS>(v, iv, vv, TB_FT_OPT_V_SCALE, false, false);
    if (sc.lerp) {
        pv = lerp_four(pv, slow[iv], sc.alpha);
        slow[iv] = pv;
    }
    w[iv] = pv;
    // newest rows first: they are the ones most likely still in L2
#pragma unroll 4
    for (int kb = KB - 1; kb >= 0; --kb) {
        const size_t i = (size_t)(kb * pi + vr) * row4 + c;
        const float4 p = w[i];
        const float4 f = make_float4(p.x + pv.x, p.y + pv.y, p.z + pv.z, p.w + pv.w);
        if (HC) __stcs(static_cast<uint2*>(comb) + i, pack_h4(f));
        else __stcs(static_cast<float4*>(comb) + i, f);
    }
}

// The same work in two kinds of launches, for the data-parallel pipeline in which the gradient rows arrive king bucket
// range by king bucket range: k_radam_factorized_rows updates the real rows of the buckets [kb0, kb1) and carries the
// running gradient sum of every virtual row through that row's gradient cell (ranges must be given in ascending
// order, so the sum is added up in the order of the fused kernel), k_radam_factorized_fold then updates the virtual
// rows and writes the folded table.  Results are bit-identical to the fused kernel.
template <bool HS, bool GS>
__global__ void __launch_bounds__(1024) k_radam_factorized_rows(float4* __restrict__ w, void* __restrict__ m, void* __restrict__ v,
                                                                 float4* __restrict__ g, float4* __restrict__ slow, int N, int pi,
                                                                 int row4, int kb0, int kb1, OptScalars sc) {
    const int vr = blockIdx.x;
    const int c = threadIdx.x;
    const float rate = sc.lr * sc.step_size;
    const float decay_mul = 1.0f - sc.decay * rate;
    const float inv_ms = 1.0f / TB_FT_OPT_M_SCALE, inv_vs = 1.0f / TB_FT_OPT_V_SCALE;
    const size_t iv = (size_t)(N + vr) * row4 + c;
    float4 gsum = kb0 == 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : g[iv];
#pragma unroll 4
    for (int kb = kb0; kb < kb1; ++kb) {
        const size_t i = (size_t)(kb * pi + vr) * row4 + c;
        float4 gi = __ldcs(g + i);
        if (GS) gi = scale4(gi, sc.grad_scale);
        float4 mi = load_moment<HS>(m, i, inv_ms, true), vi = load_moment<HS>(v, i, inv_vs, true);
        float4 p = radam_four(w[i], mi, vi, gi, sc, rate, decay_mul);
        store_moment<HS>(m, i, mi, TB_FT_OPT_M_SCALE, true, true);
        store_moment<HS>(v, i, vi, TB_FT_OPT_V_SCALE, false, true);
        if (sc.lerp) {
            p = lerp_four(p, __ldcs(slow + i), sc.alpha);
            __stcs(slow + i, p);
        }
        w[i] = p;
        gsum.x += gi.x; gsum.y += gi.y; gsum.z += gi.z; gsum.w += gi.w;
    }
    g[iv] = gsum;
}

template <bool HS, bool HC>
__global__ void __launch_bounds__(1024) k_radam_factorized_fold(float4* __restrict__ w, void* __restrict__ m, void* __restrict__ v,
                                                                 float4* __restrict__ g, float4* __restrict__ slow,
                                                                 void* __restrict__ comb, int N, int pi, int row4, OptScalars sc) {
    const int vr = blockIdx.x;
    const int c = threadIdx.x;
    const float rate = sc.lr * sc.step_size;
    const float decay_mul = 1.0f - sc.decay * rate;
    const int KB = N / pi;
    const size_t iv = (size_t)(N + vr) * row4 + c;
    float4 mv = load_moment<HS>(m, iv, 1.0f / TB_FT_OPT_M_SCALE, false), vv = load_moment<HS>(v, iv, 1.0f / TB_FT_OPT_V_SCALE, false);
    float4 pv = radam_four(w[iv], mv, vv, g[iv], sc, rate, decay_mul);
    store_moment<HS>(m, iv, mv, TB_FT_OPT_M_SCALE, true, false);
    store_moment<HS>(v, iv, vv, TB_FT_OPT_V_SCALE, false, false);
    if (sc.lerp) {
        pv = lerp_four(pv, slow[iv], sc.alpha);
        slow[iv] = pv;
    }
    w[iv] = pv;
#pragma unroll 4
    for (int kb = 0; kb < KB; ++kb) {
        const size_t i = (size_t)(kb * pi + vr) * row4 + c;
        const float4 p = __ldcs(w + i);
        const float4 f = make_float4(p.x + pv.x, p.y + pv.y, p.z + pv.z, p.w + pv.w);
        if (HC) __stcs(static_cast<uint2*>(comb) + i, pack_h4(f));
        else __stcs(static_cast<float4*>(comb) + i, f);
    }
}

int launch_radam_factorized_rows(cudaStream_t s, float* w, void* m, void* v, float* g, float* slow, int N, int pi, int F, int kb0,
                                 int kb1, OptScalars sc, int half_state) {
    float4 *w4 = reinterpret_cast<float4*>(w), *g4 = reinterpret_cast<float4*>(g), *s4 = reinterpret_cast<float4*>(slow);
    const bool gs = sc.grad_scale != 1.0f;
#define ROWS(HS, GS) k_radam_factorized_rows<HS, GS><<<pi, F / 4, 0, s>>>(w4, m, v, g4, s4, N, pi, F / 4, kb0, kb1, sc)
    if (half_state) { if (gs) ROWS(true, true); else ROWS(true, false); }
    else { if (gs) ROWS(false, true); else ROWS(false, false); }
#undef ROWS
    return 1;
}

int launch_radam_factorized_fold(cudaStream_t s, float* w, void* m, void* v, float* g, float* slow, void* comb, int N, int pi,
                                 int F, OptScalars sc, int half_state, int half_comb) {
    float4 *w4 = reinterpret_cast<float4*>(w), *g4 = reinterpret_cast<float4*>(g), *s4 = reinterpret_cast<float4*>(slow);
#define FOLD(HS, HC) k_radam_factorized_fold<HS, HC><<<pi, F / 4, 0, s>>>(w4, m, v, g4, s4, comb, N, pi, F / 4, sc)
    if (half_state) { if (half_comb) FOLD(true, true); else FOLD(true, false); }
    else { if (half_comb) FOLD(false, true); else FOLD(false, false); }
#undef FOLD
    return 1;
}

int launch_radam_factorized(cudaStream_t s, float* w, void* m, void* v, float* g, float* slow, void* comb, int N,
                            int pi, int F, OptScalars sc, int half_state, int half_comb) {
    float4 *w4 = reinterpret_cast<float4*>(w), *g4 = reinterpret_cast<float4*>(g), *s4 = reinterpret_cast<float4*>(slow);
#define FUSED(T, MB, HS, HC) k_radam_factorized<T, MB, HS, HC><<<pi, F / 4, 0, s>>>(w4, m, v, g4, s4, comb, N, pi, F / 4, sc)
    if (F / 4 <= 384) {
        if (half_state) { if (half_comb) FUSED(384, 3, true, true); else FUSED(384, 3, true, false); }
        else { if (half_comb) FUSED(384, 3, false, true); else FUSED(384, 3, false, false); }
    } else {
        if (half_state) { if (half_comb) FUSED(1024, 1, true, true); else FUSED(1024, 1, true, false); }
        else { if (half_comb) FUSED(1024, 1, false, true); else FUSED(1024, 1, false, false); }
    }
#undef FUSED
    return 1;
}
