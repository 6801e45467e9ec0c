// Hidden-layer kernels: bucket grouping of the batch, the L1 contraction (per-bucket + shared, or the
// Simple architecture's single matrix), the fused tail (L1 activation .. L2 .. L3 .. loss and its
// backward to the L1 output), the small-layer weight gradients, the L1 weight gradient and the fused
// L1 input gradient + FT activation gradient.
//
// Positions are never physically permuted.  `order` lists the positions grouped by LayerStack bucket
// (stable), `tiles` cuts it into runs of at most TB_TILE_M positions of one bucket; kernels gather
// rows through `order` and write results back at the position's own row.
#include "common.cuh"

// asynchronous 16-byte copy global -> shared (both 16-byte aligned)
static __device__ __forceinline__ void dg_cp16(void* dst_shared, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}

// asynchronous 8-byte copy global -> shared (both 8-byte aligned)
static __device__ __forceinline__ void dg_cp8(void* dst_shared, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src) : "memory");
}

#include <cuda_fp16.h>
#include <stdlib.h>

#include <type_traits>

static __device__ __forceinline__ unsigned dk_pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
}
static __device__ __forceinline__ float2 dk_unpack_h2(unsigned pair) { return __half22float2(*reinterpret_cast<const __half2*>(&pair)); }
// native_clamp_half (native_kernels.cu:636-646): values beyond the fp16 range are clamped and counted
static __device__ __forceinline__ float clamp_half_count(float v, unsigned& clamps) {
    if (v > 65504.0f) { ++clamps; return 65504.0f; }
    if (v < -65504.0f) { ++clamps; return -65504.0f; }
    return v;
}

#define FT_POST_SCALE (127.0f / 128.0f)  // bins/nnue_train/src/arch.rs:64-70
#define L1_SQR_SCALE (127.0f / 128.0f)

// ------------------------------------------------------------------------------------------------
// L1 forward.  y[pos, o] = (bb[g, o] + sum_k x[pos, k] wb[g, o, k]) + (bs[o] + sum_k x[pos, k] ws[k, o])
// (dense_mm_bucket.rs:45-73 + dense_mm.rs:37-54 + elementwise add, trainer_layerstack.rs:2373-2530).
// Without buckets (Simple) only the second term exists.  One block per tile, K in chunks of 64.
// ------------------------------------------------------------------------------------------------
template <bool HAS_BUCKET>
__global__ void __launch_bounds__(256) k_l1_forward(const float* __restrict__ x, int K, const int* __restrict__ order,
                                                     const TileDesc* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                     const float* __restrict__ wb, const float* __restrict__ bb,
                                                     const float* __restrict__ ws, const float* __restrict__ bs,
                                                     float* __restrict__ y, int l1, int nb) {
    if ((int)blockIdx.x >= *n_tiles) return;
    const TileDesc td = tiles[blockIdx.x];
    __shared__ float xs[TB_TILE_M][65];
    __shared__ float wbs[TB_MAX_L1][65];
    __shared__ float wss[64][TB_MAX_L1 + 1];
    __shared__ int s_pos[TB_TILE_M];
    const int tid = threadIdx.x;
    if (tid < TB_TILE_M) s_pos[tid] = tid < td.count ? order[td.start + tid] : -1;
    const int p = tid >> 3, og = tid & 7;
    const bool use_b = HAS_BUCKET && td.bucket < nb;
    float accb[4] = {0.f, 0.f, 0.f, 0.f}, accs[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += 64) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int e = tid + 256 * j;
            const int r = e >> 6, c = e & 63;
            const int pos = s_pos[r];
            xs[r][c] = pos >= 0 ? x[(size_t)pos * K + k0 + c] : 0.f;
        }
        if (use_b)
            for (int e = tid; e < l1 * 64; e += 256) {
                const int o = e >> 6, c = e & 63;
                wbs[o][c] = wb[((size_t)td.bucket * l1 + o) * K + k0 + c];
            }
        for (int e = tid; e < 64 * l1; e += 256) {
            const int kk = e / l1, o = e - kk * l1;
            wss[kk][o] = ws[(size_t)k0 * l1 + e];
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 64; ++kk) {
            const float xv = xs[p][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int o = og + 8 * j;
                if (o < l1) {
                    if (use_b) accb[j] += xv * wbs[o][kk];
                    accs[j] += xv * wss[kk][o];
                }
            }
        }
    }
    const int pos = s_pos[p];
    if (pos < 0) return;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int o = og + 8 * j;
        if (o < l1) {
            const float ys = bs[o] + accs[j];
            if (HAS_BUCKET) {
                const float yb = use_b ? bb[td.bucket * l1 + o] + accb[j] : 0.f;
                y[(size_t)pos * l1 + o] = yb + ys;
            } else {
                y[(size_t)pos * l1 + o] = ys;
            }
        }
    }
}

// Register-tiled variant for l1 % 4 == 0 (every shipped configuration).  A block of 64 threads owns one tile
// of 32 positions and all NOUT output columns (LayerStack: [0, l1) per-bucket, [l1, 2 l1) shared; Simple:
// [0, l1)), NT = ceil(NOUT / 32) column tiles.  Thread (ty, tx) accumulates rows 4ty..4ty+3 x columns
// 4tx..4tx+3 of every column tile; per k it needs one 128-bit load of x (stored k-major in shared memory) and
// one per column tile of w.  The next K chunk is fetched into registers while the current one is multiplied.
template <int NT, bool HAS_BUCKET>
__global__ void __launch_bounds__(64) k_l1_forward_tiled(const float* __restrict__ x, int K, const int* __restrict__ order,
                                                          const TileDesc* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                          const float* __restrict__ wb, const float* __restrict__ bb,
                                                          const float* __restrict__ ws, const float* __restrict__ bs,
                                                          float* __restrict__ y, int l1, int nb) {
    if ((int)blockIdx.x >= *n_tiles) return;
    const TileDesc td = tiles[blockIdx.x];
    constexpr int WS_LD = NT * 32 + 4;
    __shared__ __align__(16) float xs[32][36];      // [k][position]
    __shared__ __align__(16) float wsm[32][WS_LD];  // [k][output column]
    __shared__ int s_pos[TB_TILE_M];
    const int tid = threadIdx.x;
    const int ty = tid >> 3, tx = tid & 7;
    const bool use_b = HAS_BUCKET && td.bucket < nb;
    const int NOUT = HAS_BUCKET ? 2 * l1 : l1;
    if (tid < TB_TILE_M) s_pos[tid] = tid < td.count ? order[td.start + tid] : -1;
    for (int e = tid; e < 32 * WS_LD; e += 64) (&wsm[0][0])[e] = 0.f;  // columns >= NOUT stay zero
    __syncthreads();

    // global -> register staging of one K chunk
    float4 xr[4];
    float4 wr[NT * 4];
    const int l1q = l1 >> 2;  // float4 per shared-weight row
    auto fetch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = tid + 64 * j;
            const int row = e >> 3, k4 = (e & 7) << 2;
            const int pos = s_pos[row];
            xr[j] = pos >= 0 ? __ldg(reinterpret_cast<const float4*>(x + (size_t)pos * K + k0 + k4)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < NT * 4; ++j) {
            const int e = tid + 64 * j;  // float4 index inside the chunk's weights
            wr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (HAS_BUCKET) {
                // first l1 * 8 float4: per-bucket rows wb[g][o][k0 + k4 ..]; then 32 * l1q float4: shared rows ws[k][o4 ..]
                if (e < l1 * 8) {
                    if (use_b) {
                        const int o = e >> 3, k4 = (e & 7) << 2;
                        wr[j] = __ldg(reinterpret_cast<const float4*>(wb + ((size_t)td.bucket * l1 + o) * K + k0 + k4));
                    }
                } else if (e < l1 * 8 + 32 * l1q) {
                    wr[j] = __ldg(reinterpret_cast<const float4*>(ws + (size_t)k0 * l1) + (e - l1 * 8));
                }
            } else if (e < 32 * l1q) {
                wr[j] = __ldg(reinterpret_cast<const float4*>(ws + (size_t)k0 * l1) + e);
            }
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = tid + 64 * j;
            const int row = e >> 3, k4 = (e & 7) << 2;
            xs[k4 + 0][row] = xr[j].x; xs[k4 + 1][row] = xr[j].y; xs[k4 + 2][row] = xr[j].z; xs[k4 + 3][row] = xr[j].w;
        }
#pragma unroll
        for (int j = 0; j < NT * 4; ++j) {
            const int e = tid + 64 * j;
            if (HAS_BUCKET) {
                if (e < l1 * 8) {
                    const int o = e >> 3, k4 = (e & 7) << 2;
                    wsm[k4 + 0][o] = wr[j].x; wsm[k4 + 1][o] = wr[j].y; wsm[k4 + 2][o] = wr[j].z; wsm[k4 + 3][o] = wr[j].w;
                } else if (e < l1 * 8 + 32 * l1q) {
                    const int r = e - l1 * 8;
                    const int k = r / l1q, o4 = (r - k * l1q) << 2;
                    *reinterpret_cast<float4*>(&wsm[k][l1 + o4]) = wr[j];
                }
            } else if (e < 32 * l1q) {
                const int k = e / l1q, o4 = (e - k * l1q) << 2;
                *reinterpret_cast<float4*>(&wsm[k][o4]) = wr[j];
            }
        }
    };

    float acc[NT][4][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[t][i][j] = 0.f;

    fetch(0);
    for (int k0 = 0; k0 < K; k0 += 32) {
        __syncthreads();  // the previous chunk has been consumed
        stage();
        __syncthreads();
        if (k0 + 32 < K) fetch(k0 + 32);
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[k][4 * ty]);
            const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float4 b = *reinterpret_cast<const float4*>(&wsm[k][t * 32 + 4 * tx]);
                const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[t][i][j] += av[i] * bv[j];
            }
        }
    }
    // combine the two halves through shared memory: out[row][col]
    __syncthreads();
    float* outs = &wsm[0][0];  // [32][WS_LD]
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<float4*>(&outs[(4 * ty + i) * WS_LD + t * 32 + 4 * tx]) =
                make_float4(acc[t][i][0], acc[t][i][1], acc[t][i][2], acc[t][i][3]);
    __syncthreads();
    for (int e = tid; e < TB_TILE_M * l1; e += 64) {
        const int r = e / l1, o = e - r * l1;
        const int pos = s_pos[r];
        if (pos < 0) continue;
        if (HAS_BUCKET) {
            const float yb = use_b ? bb[td.bucket * l1 + o] + outs[r * WS_LD + o] : 0.f;
            const float ysv = bs[o] + outs[r * WS_LD + l1 + o];
            y[(size_t)pos * l1 + o] = yb + ysv;
        } else {
            y[(size_t)pos * l1 + o] = bs[o] + outs[r * WS_LD + o];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// L1 forward, streaming form for l1 = 8, 16 or 32.  The per-bucket and the shared layer see the same input and their
// outputs are added, so they are one contraction with the effective weights weff[g] = wb[g] + ws^T (weff[nb] = ws^T for
// positions without a bucket), built once per step by k_l1_weff.  A block owns 128 consecutive positions of the bucket
// order (half a work unit); x rows and the weight rows arrive in K chunks of 16 through a three-stage ring of
// asynchronous copies; a thread keeps a 4-position x 8-output tile of sums in registers and reads both operands as
// 128-bit rows along k (row stride 20 floats: the rows a quarter warp touches fall into different banks).
// ------------------------------------------------------------------------------------------------
__global__ void k_l1_weff(const float* __restrict__ wb, const float* __restrict__ bb, const float* __restrict__ ws,
                          const float* __restrict__ bs, int K, int l1, int nb, float* __restrict__ weff, float* __restrict__ beff) {
    const int g = blockIdx.y;
    const size_t n = (size_t)l1 * K;
    const bool use_b = wb != nullptr && g < nb;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int o = (int)(i / K), k = (int)(i - (size_t)o * K);
        float v = ws[(size_t)k * l1 + o];
        if (use_b) v = wb[(size_t)g * n + i] + v;
        weff[(size_t)g * n + i] = v;
    }
    if (blockIdx.x == 0 && (int)threadIdx.x < l1) {
        float b = bs ? bs[threadIdx.x] : 0.f;
        if (use_b && bb) b = bb[(size_t)g * l1 + threadIdx.x] + b;
        beff[(size_t)g * l1 + threadIdx.x] = b;
    }
}

#define LF_POS 128
#define LF_KC 16
#define LF_LD 20
#define LF_STAGES 3
static_assert(2 * LF_POS == TB_UNIT_TILES * TB_TILE_M, "a block of the streaming forward owns half a work unit");
template <int L1>
__global__ void __launch_bounds__(4 * L1) k_l1_forward_stream(const float* __restrict__ x, int K, const int* __restrict__ order,
                                                              const TileDesc* __restrict__ tiles, const TileDesc* __restrict__ units,
                                                              const int* __restrict__ n_units, const float* __restrict__ weff,
                                                              const float* __restrict__ beff, float* __restrict__ y, int nb) {
    constexpr int TX = L1 / 8, TY = 32 / TX, NT = 32 * TX;
    constexpr int STAGE_FLOATS = (LF_POS + L1) * LF_LD;
    extern __shared__ __align__(16) float s_ring[];  // [LF_STAGES][LF_POS + L1][LF_LD]
    __shared__ int s_pos[LF_POS];
    const int u = blockIdx.x >> 1, h = blockIdx.x & 1;
    if (u >= *n_units) return;
    const TileDesc ud = units[u];
    const int per = LF_POS / TB_TILE_M;
    const int first = ud.start + h * per, last = min(ud.start + ud.count, first + per);
    if (first >= last) return;
    const int p_begin = tiles[first].start;
    const int n = tiles[last - 1].start + tiles[last - 1].count - p_begin;
    const int g = ud.bucket < nb ? ud.bucket : nb;
    const int tid = threadIdx.x;
    for (int i = tid; i < LF_POS; i += NT) s_pos[i] = order[p_begin + (i < n ? i : 0)];  // rows past the end repeat the first
    __syncthreads();
    const float* __restrict__ wg = weff + (size_t)g * L1 * K;
    const int nk = K / LF_KC;
    auto issue = [&](int it) {
        if (it < nk) {
            float* st = s_ring + (size_t)(it % LF_STAGES) * STAGE_FLOATS;
            const int k0 = it * LF_KC;
            for (int e = tid; e < LF_POS * 4; e += NT) {
                const int r = e >> 2, pc = e & 3;
                dg_cp16(st + r * LF_LD + 4 * pc, x + (size_t)s_pos[r] * K + k0 + 4 * pc);
            }
            for (int e = tid; e < L1 * 4; e += NT) {
                const int o = e >> 2, pc = e & 3;
                dg_cp16(st + (LF_POS + o) * LF_LD + 4 * pc, wg + (size_t)o * K + k0 + 4 * pc);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int lane = tid & 31, warp = tid >> 5;
    const int tx = lane % TX, ty = lane / TX;
    const int row0 = warp * (4 * TY) + ty;  // the thread's positions: row0 + TY * i
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int it = 0; it < LF_STAGES - 1; ++it) issue(it);
    for (int it = 0; it < nk; ++it) {
        asm volatile("cp.async.wait_group %0;" ::"n"(LF_STAGES - 2) : "memory");
        __syncthreads();  // chunk `it` has landed for every thread; chunk it - 1 has been consumed by every thread
        issue(it + LF_STAGES - 1);
        const float* st = s_ring + (size_t)(it % LF_STAGES) * STAGE_FLOATS;
#pragma unroll
        for (int kk = 0; kk < LF_KC; kk += 4) {
            float4 xv[4], wv[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = *reinterpret_cast<const float4*>(st + (row0 + TY * i) * LF_LD + kk);
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = *reinterpret_cast<const float4*>(st + (LF_POS + tx + TX * j) * LF_LD + kk);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[i][j] += xv[i].x * wv[j].x;
                    acc[i][j] += xv[i].y * wv[j].y;
                    acc[i][j] += xv[i].z * wv[j].z;
                    acc[i][j] += xv[i].w * wv[j].w;
                }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + TY * i;
        if (r >= n) continue;
        float* yr = y + (size_t)s_pos[r] * L1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int o = tx + TX * j;
            yr[o] = acc[i][j] + beff[(size_t)g * L1 + o];
        }
    }
}

int launch_l1_forward(cudaStream_t s, const float* x, int K, const int* order, const TileDesc* tiles,
                      const int* n_tiles, int max_tiles, const float* wb, const float* bb, const float* ws,
                      const float* bs, float* y, int l1, int nb, float* weff, int tf32, int* error_flag) {
    if ((l1 == 8 || l1 == 16 || l1 == 32) && K % LF_KC == 0 && weff != nullptr) {
        float* beff = weff + (size_t)(nb + 1) * l1 * K;
        k_l1_weff<<<dim3(ceil_div(l1 * K, 256 * 4), nb + 1), 256, 0, s>>>(wb, bb, ws, bs, K, l1, wb ? nb : 0, weff, beff);
        if (tf32 && error_flag && l1_forward_tc_supported(K, l1))
            return 1 + launch_l1_forward_tc(s, x, K, order, tiles, n_tiles, max_tiles, weff, beff, y, l1, wb ? nb : 0, error_flag);
        const int max_units = sort_max_units(max_tiles);
        const size_t smem = (size_t)LF_STAGES * (LF_POS + l1) * LF_LD * sizeof(float);
        const TileDesc* units = tiles + max_tiles;
        const int nbe = wb ? nb : 0;
        if (l1 == 8) k_l1_forward_stream<8><<<2 * max_units, 32, smem, s>>>(x, K, order, tiles, units, n_tiles + 1, weff, beff, y, nbe);
        else if (l1 == 16) k_l1_forward_stream<16><<<2 * max_units, 64, smem, s>>>(x, K, order, tiles, units, n_tiles + 1, weff, beff, y, nbe);
        else k_l1_forward_stream<32><<<2 * max_units, 128, smem, s>>>(x, K, order, tiles, units, n_tiles + 1, weff, beff, y, nbe);
        return 2;
    }
    const int nout = wb ? 2 * l1 : l1;
    if (l1 % 4 == 0 && nout <= 64) {
        if (wb) {
            if (nout <= 32) k_l1_forward_tiled<1, true><<<max_tiles, 64, 0, s>>>(x, K, order, tiles, n_tiles, wb, bb, ws, bs, y, l1, nb);
            else k_l1_forward_tiled<2, true><<<max_tiles, 64, 0, s>>>(x, K, order, tiles, n_tiles, wb, bb, ws, bs, y, l1, nb);
        } else {
            k_l1_forward_tiled<1, false><<<max_tiles, 64, 0, s>>>(x, K, order, tiles, n_tiles, wb, bb, ws, bs, y, l1, nb);
        }
        return 1;
    }
    if (wb)
        k_l1_forward<true><<<max_tiles, 256, 0, s>>>(x, K, order, tiles, n_tiles, wb, bb, ws, bs, y, l1, nb);
    else
        k_l1_forward<false><<<max_tiles, 256, 0, s>>>(x, K, order, tiles, n_tiles, wb, bb, ws, bs, y, l1, nb);
    return 1;
}

// ------------------------------------------------------------------------------------------------
// loss (pointwise/loss_wdl.rs:63-88, pointwise/loss_wrm.rs:99-180 default path)
// ------------------------------------------------------------------------------------------------
static __device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// the extended WRM loss's per-position weight (loss_wrm / wrm_weight_sum, native_kernels.cu:455-458, 538-543)
static __device__ __forceinline__ float wrm_weight(const LossParams& lp, float target_wrm) {
    const float wb = (target_wrm - 0.5f) * (target_wrm - 0.5f) * target_wrm * (1.0f - target_wrm);
    return 1.0f + (powf(2.0f, lp.w1) - 1.0f) * powf(wb, lp.w2);
}

// returns the position's contribution to the reported loss sum (err^2 for the plain losses) and its output gradient
static __device__ __forceinline__ double loss_point(const LossParams& lp, float out, float score, float wdl, float* dy) {
    if (lp.kind == 0) {
        const float p = sigmoidf_(out * lp.scale);
        const float ys = sigmoidf_(score * lp.scale);
        const float y = lp.lambda * wdl + (1.0f - lp.lambda) * ys;
        const float err = p - y;
        *dy = 2.0f * err * p * (1.0f - p) * lp.scale * lp.norm;
        return (double)err * (double)err;
    }
    const float pt = (score - lp.target_offset) / lp.target_scaling;
    const float pmt = (-score - lp.target_offset) / lp.target_scaling;
    const float target_wrm = 0.5f * (1.0f + sigmoidf_(pt) - sigmoidf_(pmt));
    const float target = lp.lambda * wdl + (1.0f - lp.lambda) * target_wrm;
    const float scorenet = out * lp.nnue2score;
    const float q = sigmoidf_((scorenet - lp.in_offset) / lp.in_scaling);
    const float qm = sigmoidf_((-scorenet - lp.in_offset) / lp.in_scaling);
    const float qf = 0.5f * (1.0f + q - qm);
    const float err = qf - target;
    if (!lp.extended) {
        *dy = err * (lp.nnue2score / lp.in_scaling) * (q * (1.0f - q) + qm * (1.0f - qm)) * lp.norm;
        return (double)err * (double)err;
    }
    // loss_wrm, extended branch (native_kernels.cu:454-474): |err|^pow_exp, asymmetry above the target, weights
    // normalised by their sum over the batch (which replaces the per-position normaliser)
    const float weight = wrm_weight(lp, target_wrm);
    const float asym = qf > target ? 1.0f + lp.qp_asymmetry : 1.0f;
    const float abs_err = fabsf(err);
    const float abs_pow = powf(abs_err, lp.pow_exp - 1.0f);
    const float signed_pow = err < 0.0f ? -abs_pow : abs_pow;
    const float inv_wsum = (float)(1.0 / *lp.weight_sum);
    const float pred_grad = 0.5f * (lp.nnue2score / lp.in_scaling) * (q * (1.0f - q) + qm * (1.0f - qm));
    *dy = (weight * inv_wsum) * (asym * lp.pow_exp * signed_pow) * pred_grad;
    return (double)(asym * powf(abs_err, lp.pow_exp) * weight * lp.n_pos * inv_wsum);
}

__global__ void __launch_bounds__(256) k_wrm_weight_partials(const float* __restrict__ score, int B, LossParams lp,
                                                             double* __restrict__ partials) {
    __shared__ double s[256];
    const int b = blockIdx.x * 256 + threadIdx.x;
    double w = 0.0;
    if (b < B) {
        const float sc = score[b];
        const float tp = sigmoidf_((sc - lp.target_offset) / lp.target_scaling), tn = sigmoidf_((-sc - lp.target_offset) / lp.target_scaling);
        w = (double)wrm_weight(lp, 0.5f * (1.0f + tp - tn));
    }
    s[threadIdx.x] = w;
    __syncthreads();
    for (int d = 128; d > 0; d >>= 1) {
        if ((int)threadIdx.x < d) s[threadIdx.x] += s[threadIdx.x + d];
        __syncthreads();
    }
    if (threadIdx.x == 0) partials[blockIdx.x] = s[0];
}

// sum of err^2 over the block in f64, one partial per block (fixed order: no atomics)
static __device__ __forceinline__ void block_loss_partial(double v, double* partials) {
    __shared__ double s_w[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_down_sync(0xffffffffu, v, d);
    if (lane == 0) s_w[w] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        const int nw = (blockDim.x + 31) >> 5;
        for (int i = 0; i < nw; ++i) t += s_w[i];
        partials[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256) k_reduce_double(const double* __restrict__ partials, int n, double* __restrict__ out) {
    __shared__ double s[256];
    double t = 0.0;
    for (int i = threadIdx.x; i < n; i += 256) t += partials[i];
    s[threadIdx.x] = t;
    __syncthreads();
    for (int d = 128; d > 0; d >>= 1) {
        if ((int)threadIdx.x < d) s[threadIdx.x] += s[threadIdx.x + d];
        __syncthreads();
    }
    if (threadIdx.x == 0) *out = s[0];
}

// ------------------------------------------------------------------------------------------------
// LayerStack tail, one thread per position (trainer_layerstack.rs:2530-2717 forward,
// :2976-3325 backward): l1_total -> main / skip -> sqr, concat, CReLU -> L2 -> CReLU -> L3 -> + skip ->
// loss, then back to dl1_total.  Keeps l2_input, dl2_out, l2_acted for the weight gradients.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_tail_layerstack(const float* __restrict__ l1_total, const int* __restrict__ bucket,
                                                          const float* __restrict__ score, const float* __restrict__ wdl,
                                                          const float* __restrict__ l2_w, const float* __restrict__ l2_b,
                                                          const float* __restrict__ l3_w, const float* __restrict__ l3_b,
                                                          LossParams lp, int B, int l1, int l2, int nb,
                                                          float* __restrict__ net_output, float* __restrict__ dy_out,
                                                          float* __restrict__ dl1_total, float* __restrict__ l2_input_o,
                                                          float* __restrict__ dl2_out_o, float* __restrict__ l2_acted_o,
                                                          double* __restrict__ loss_partials, int backward) {
    extern __shared__ float s_w[];
    const int l1e = l1 - 1, l2in = 2 * l1e;
    float* sw2 = s_w;                      // [nb][l2][l2in]
    float* sb2 = sw2 + nb * l2 * l2in;     // [nb][l2]
    float* sw3 = sb2 + nb * l2;            // [nb][l2]
    float* sb3 = sw3 + nb * l2;            // [nb]
    for (int i = threadIdx.x; i < nb * l2 * l2in; i += blockDim.x) sw2[i] = l2_w[i];
    for (int i = threadIdx.x; i < nb * l2; i += blockDim.x) { sb2[i] = l2_b[i]; sw3[i] = l3_w[i]; }
    for (int i = threadIdx.x; i < nb; i += blockDim.x) sb3[i] = l3_b[i];
    __syncthreads();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    double e2 = 0.0;
    if (b < B) {
        const int g = bucket[b];
        const bool valid = (unsigned)g < (unsigned)nb;
        float pre[2 * TB_MAX_L1], in[2 * TB_MAX_L1], d2[TB_MAX_L2], a2[TB_MAX_L2];
        float mainv[TB_MAX_L1];
        for (int i = 0; i < l1e; ++i) {
            const float m = l1_total[(size_t)b * l1 + i];
            mainv[i] = m;
            pre[i] = m * m * L1_SQR_SCALE;
            pre[l1e + i] = m;
        }
        const float skip = l1_total[(size_t)b * l1 + l1e];
        for (int i = 0; i < l2in; ++i) in[i] = crelu01(pre[i]);
        float l3 = 0.f;
        if (valid) {
            for (int o = 0; o < l2; ++o) {
                const float* wr = sw2 + ((size_t)g * l2 + o) * l2in;
                float sum = sb2[g * l2 + o];
                for (int i = 0; i < l2in; ++i) sum += in[i] * wr[i];
                d2[o] = sum;
            }
            for (int o = 0; o < l2; ++o) a2[o] = crelu01(d2[o]);
            l3 = sb3[g];
            for (int o = 0; o < l2; ++o) l3 += a2[o] * sw3[g * l2 + o];
        } else {
            for (int o = 0; o < l2; ++o) { d2[o] = 0.f; a2[o] = 0.f; }
        }
        const float out = l3 + skip;
        float dyv;
        e2 = loss_point(lp, out, score[b], wdl[b], &dyv);
        net_output[b] = out;
        dy_out[b] = dyv;
        if (backward) {
            float dl2o[TB_MAX_L2];
            for (int o = 0; o < l2; ++o) {
                const float da = valid ? dyv * sw3[g * l2 + o] : 0.f;
                dl2o[o] = (d2[o] > 0.f && d2[o] < 1.0f) ? da : 0.f;
            }
            for (int i = 0; i < l2in; ++i) {
                float sum = 0.f;
                if (valid)
                    for (int o = 0; o < l2; ++o) sum += dl2o[o] * sw2[((size_t)g * l2 + o) * l2in + i];
                // crelu_grad on l2_pre, then concat split: first half is d(sqr), second half d(main)
                pre[i] = (pre[i] > 0.f && pre[i] < 1.0f) ? sum : 0.f;
            }
            for (int i = 0; i < l1e; ++i) {
                const float from_sqr = 2.0f * mainv[i] * L1_SQR_SCALE * pre[i];
                dl1_total[(size_t)b * l1 + i] = pre[l1e + i] + from_sqr;
            }
            dl1_total[(size_t)b * l1 + l1e] = dyv;
            for (int i = 0; i < l2in; ++i) l2_input_o[(size_t)b * l2in + i] = in[i];
            for (int o = 0; o < l2; ++o) {
                dl2_out_o[(size_t)b * l2 + o] = dl2o[o];
                l2_acted_o[(size_t)b * l2 + o] = a2[o];
            }
        }
    }
    block_loss_partial(e2, loss_partials);
}

// Warp-per-position variant for l2 <= 32 and 2 (l1 - 1) <= 32: lane o owns output o of L2, lane i input i.  Shared
// memory holds every bucket's L2 weights by output row with a row stride of TW_LD floats (rows 16-byte aligned, eight
// neighbouring rows in different banks), and a 32-float vector per warp through which a position's L2 input and L2
// output gradient reach all lanes with 128-bit broadcast loads; the forward reads a weight row with 128-bit loads, the
// backward a weight column.  Sums over the L2 inputs / outputs run in index order, like the
// oracle; only the 32-term L3 dot product is a butterfly reduction.
#define TW_LD 36
__global__ void __launch_bounds__(256) k_tail_layerstack_warp(const float* __restrict__ l1_total, const int* __restrict__ bucket,
                                                               const float* __restrict__ score, const float* __restrict__ wdl,
                                                               const float* __restrict__ l2_w, const float* __restrict__ l2_b,
                                                               const float* __restrict__ l3_w, const float* __restrict__ l3_b,
                                                               LossParams lp, int B, int l1, int l2, int nb,
                                                               float* __restrict__ net_output, float* __restrict__ dy_out,
                                                               float* __restrict__ dl1_total, float* __restrict__ l2_input_o,
                                                               float* __restrict__ dl2_out_o, float* __restrict__ l2_acted_o,
                                                               double* __restrict__ loss_partials, int backward) {
    extern __shared__ __align__(16) float s_w[];
    const int l1e = l1 - 1, l2in = 2 * l1e;
    float* swr = s_w;                            // [nb][32 outputs][TW_LD]: swr[g][o][i] = l2_w[g][o][i], zero padded
    float* sb2 = swr + (size_t)nb * 32 * TW_LD;  // [nb][l2]
    float* sw3 = sb2 + nb * l2;               // [nb][l2]
    float* sb3 = sw3 + nb * l2;               // [nb]
    float* svec = sb3 + ((nb + 3) & ~3);      // [warps][32]
    for (int e = threadIdx.x; e < nb * 32 * TW_LD; e += blockDim.x) {
        const int g = e / (32 * TW_LD), r = (e / TW_LD) & 31, c = e % TW_LD;
        swr[e] = (r < l2 && c < l2in) ? l2_w[((size_t)g * l2 + r) * l2in + c] : 0.f;
    }
    for (int i = threadIdx.x; i < nb * l2; i += blockDim.x) { sb2[i] = l2_b[i]; sw3[i] = l3_w[i]; }
    for (int i = threadIdx.x; i < nb; i += blockDim.x) sb3[i] = l3_b[i];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const unsigned full = 0xffffffffu;
    float* vec = svec + (threadIdx.x >> 5) * 32;
    const float4* vec4 = reinterpret_cast<const float4*>(vec);
    double e2 = 0.0;
    for (int b = blockIdx.x * wpb + (threadIdx.x >> 5); b < B; b += gridDim.x * wpb) {
        const int g = bucket[b];
        const bool valid = (unsigned)g < (unsigned)nb;
        const float t = lane < l1 ? l1_total[(size_t)b * l1 + lane] : 0.f;
        const float skip = __shfl_sync(full, t, l1e);
        // lane i < l1e: sqr_i; lane l1e + i: main_i (concat_l1sqr_main), then CReLU
        const float m = __shfl_sync(full, t, lane < l1e ? lane : (lane - l1e < l1e ? lane - l1e : 0));
        const float pre = lane < l1e ? m * m * L1_SQR_SCALE : m;
        const float in = lane < l2in ? crelu01(pre) : 0.f;
        float d2 = 0.f, a2 = 0.f, l3 = 0.f;
        if (valid) {
            __syncwarp();
            vec[lane] = in;
            __syncwarp();
            const float4* wr = reinterpret_cast<const float4*>(swr + ((size_t)g * 32 + lane) * TW_LD);
            float sum = lane < l2 ? sb2[g * l2 + lane] : 0.f;
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
                const float4 x = vec4[i4], w = wr[i4];
                sum += x.x * w.x; sum += x.y * w.y; sum += x.z * w.z; sum += x.w * w.w;
            }
            d2 = lane < l2 ? sum : 0.f;
            a2 = lane < l2 ? crelu01(d2) : 0.f;
            float part = lane < l2 ? a2 * sw3[g * l2 + lane] : 0.f;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(full, part, d);
            l3 = sb3[g] + part;
        }
        const float out = l3 + skip;
        float dyv;
        const double contrib = loss_point(lp, out, score[b], wdl[b], &dyv);
        if (lane == 0) {
            e2 += contrib;
            net_output[b] = out;
            dy_out[b] = dyv;
        }
        if (backward) {
            float dl2o = 0.f;
            if (valid && lane < l2) {
                const float da = dyv * sw3[g * l2 + lane];
                dl2o = (d2 > 0.f && d2 < 1.0f) ? da : 0.f;
            }
            float sum = 0.f;
            if (valid) {
                __syncwarp();
                vec[lane] = dl2o;
                __syncwarp();
                const float* wc = swr + (size_t)g * 32 * TW_LD + lane;  // column `lane`: neighbouring lanes, neighbouring banks
#pragma unroll
                for (int o4 = 0; o4 < 8; ++o4) {
                    const float4 x = vec4[o4];
                    sum += x.x * wc[(4 * o4 + 0) * TW_LD]; sum += x.y * wc[(4 * o4 + 1) * TW_LD];
                    sum += x.z * wc[(4 * o4 + 2) * TW_LD]; sum += x.w * wc[(4 * o4 + 3) * TW_LD];
                }
            }
            const float dpre = (lane < l2in && pre > 0.f && pre < 1.0f) ? sum : 0.f;  // crelu_grad on l2_pre
            // lane i < l1e: d(main_i) = dpre[l1e + i] + 2 main_i scale dpre[i]
            const float dmain_concat = __shfl_sync(full, dpre, lane + l1e < 32 ? lane + l1e : 0);
            const float from_sqr = 2.0f * t * L1_SQR_SCALE * dpre;
            if (lane < l1e) dl1_total[(size_t)b * l1 + lane] = dmain_concat + from_sqr;
            else if (lane == l1e) dl1_total[(size_t)b * l1 + l1e] = dyv;
            if (lane < l2in) l2_input_o[(size_t)b * l2in + lane] = in;
            if (lane < l2) {
                dl2_out_o[(size_t)b * l2 + lane] = dl2o;
                l2_acted_o[(size_t)b * l2 + lane] = a2;
            }
        }
    }
    block_loss_partial(e2, loss_partials);
}

int launch_wrm_weight_sum(cudaStream_t s, const float* score, int B, LossParams lp, double* partials, double* weight_sum) {
    const int blocks = ceil_div(B, 256);
    k_wrm_weight_partials<<<blocks, 256, 0, s>>>(score, B, lp, partials);
    k_reduce_double<<<1, 256, 0, s>>>(partials, blocks, weight_sum);
    return 2;
}

int launch_tail_layerstack(cudaStream_t s, const float* l1_total, const int* bucket, const float* score,
                           const float* wdl, const float* l2_w, const float* l2_b, const float* l3_w,
                           const float* l3_b, LossParams lp, int B, int l1, int l2, int nb, float* net_output,
                           float* dy, float* dl1_total, float* l2_input, float* dl2_out, float* l2_acted,
                           double* loss_partials, double* loss_acc, int backward) {
    const int l2in = 2 * (l1 - 1);
    const size_t smem = sizeof(float) * ((size_t)nb * l2 * l2in + 2 * (size_t)nb * l2 + nb);
    cudaFuncSetAttribute(k_tail_layerstack, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const size_t wsmem = sizeof(float) * ((size_t)nb * 32 * TW_LD + 2 * (size_t)nb * l2 + ((nb + 3) & ~3) + 8 * 32);
    if (l2 <= 32 && l2 % 4 == 0 && l2in <= 32 && wsmem <= 110 * 1024) {
        cudaFuncSetAttribute(k_tail_layerstack_warp, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        int blocks = ceil_div(B, 8);
        if (blocks > 148 * 4) blocks = 148 * 4;
        k_tail_layerstack_warp<<<blocks, 256, wsmem, s>>>(l1_total, bucket, score, wdl, l2_w, l2_b, l3_w, l3_b, lp, B, l1, l2, nb,
                                                        net_output, dy, dl1_total, l2_input, dl2_out, l2_acted, loss_partials,
                                                        backward);
        k_reduce_double<<<1, 256, 0, s>>>(loss_partials, blocks, loss_acc);
        return 2;
    }
    const int blocks = ceil_div(B, 128);
    k_tail_layerstack<<<blocks, 128, smem, s>>>(l1_total, bucket, score, wdl, l2_w, l2_b, l3_w, l3_b, lp, B, l1, l2, nb,
                                               net_output, dy, dl1_total, l2_input, dl2_out, l2_acted, loss_partials, backward);
    k_reduce_double<<<1, 256, 0, s>>>(loss_partials, blocks, loss_acc);
    return 2;
}

// ------------------------------------------------------------------------------------------------
// Simple tail (trainer_simple.rs:1281-1508 forward, :1560-1765 backward): l1_pre -> act -> L2 -> act ->
// L3 -> loss and back to dl1_pre.  l2_w is [l1][l2], l3_w [l2].
// ------------------------------------------------------------------------------------------------
static __device__ __forceinline__ float act_fwd(int act, float x) {
    const float a = crelu01(x);
    return act == 0 ? a : a * a;
}
static __device__ __forceinline__ float act_grad(int act, float x, float up) {
    if (act == 0) return (x > 0.f && x < 1.0f) ? up : 0.f;
    const float a = crelu01(x);
    return up * ((a > 0.f && a < 1.0f) ? 2.0f * a : 0.f);
}

__global__ void __launch_bounds__(128) k_tail_simple(const float* __restrict__ l1_pre, const float* __restrict__ score,
                                                      const float* __restrict__ wdl, const float* __restrict__ l2_w,
                                                      const float* __restrict__ l2_b, const float* __restrict__ l3_w,
                                                      const float* __restrict__ l3_b, LossParams lp, int act, int B, int l1,
                                                      int l2, float* __restrict__ net_output, float* __restrict__ dy_out,
                                                      float* __restrict__ dl1_pre, float* __restrict__ l1_acted_o,
                                                      float* __restrict__ dl2_pre_o, float* __restrict__ l2_acted_o,
                                                      double* __restrict__ loss_partials, int backward) {
    extern __shared__ float s_w[];
    float* sw2 = s_w;            // [l1][l2]
    float* sb2 = sw2 + l1 * l2;  // [l2]
    float* sw3 = sb2 + l2;       // [l2]
    for (int i = threadIdx.x; i < l1 * l2; i += blockDim.x) sw2[i] = l2_w[i];
    for (int i = threadIdx.x; i < l2; i += blockDim.x) { sb2[i] = l2_b[i]; sw3[i] = l3_w[i]; }
    __syncthreads();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    double e2 = 0.0;
    if (b < B) {
        float x1[TB_MAX_L1 * 2], a1[TB_MAX_L1 * 2], x2[TB_MAX_L2], a2[TB_MAX_L2];
        for (int i = 0; i < l1; ++i) { x1[i] = l1_pre[(size_t)b * l1 + i]; a1[i] = act_fwd(act, x1[i]); }
        for (int o = 0; o < l2; ++o) {
            float sum = sb2[o];
            for (int i = 0; i < l1; ++i) sum += a1[i] * sw2[i * l2 + o];
            x2[o] = sum;
            a2[o] = act_fwd(act, sum);
        }
        float out = l3_b[0];
        for (int o = 0; o < l2; ++o) out += a2[o] * sw3[o];
        float dyv;
        e2 = loss_point(lp, out, score[b], wdl[b], &dyv);
        net_output[b] = out;
        dy_out[b] = dyv;
        if (backward) {
            float d2[TB_MAX_L2];
            for (int o = 0; o < l2; ++o) d2[o] = act_grad(act, x2[o], dyv * sw3[o]);
            for (int i = 0; i < l1; ++i) {
                float sum = 0.f;
                for (int o = 0; o < l2; ++o) sum += d2[o] * sw2[i * l2 + o];
                dl1_pre[(size_t)b * l1 + i] = act_grad(act, x1[i], sum);
                l1_acted_o[(size_t)b * l1 + i] = a1[i];
            }
            for (int o = 0; o < l2; ++o) {
                dl2_pre_o[(size_t)b * l2 + o] = d2[o];
                l2_acted_o[(size_t)b * l2 + o] = a2[o];
            }
        }
    }
    block_loss_partial(e2, loss_partials);
}

// Warp-per-position variant for l1 <= 32 and l2 <= 32 (lane i: L1 output i; lane o: L2 output o).
__global__ void __launch_bounds__(256) k_tail_simple_warp(const float* __restrict__ l1_pre, const float* __restrict__ score,
                                                           const float* __restrict__ wdl, const float* __restrict__ l2_w,
                                                           const float* __restrict__ l2_b, const float* __restrict__ l3_w,
                                                           const float* __restrict__ l3_b, LossParams lp, int act, int B, int l1,
                                                           int l2, float* __restrict__ net_output, float* __restrict__ dy_out,
                                                           float* __restrict__ dl1_pre, float* __restrict__ l1_acted_o,
                                                           float* __restrict__ dl2_pre_o, float* __restrict__ l2_acted_o,
                                                           double* __restrict__ loss_partials, int backward) {
    __shared__ float sw2[32][33];   // [i][o]
    __shared__ float sw2t[32][33];  // [o][i]
    __shared__ float sb2[32], sw3[32];
    for (int e = threadIdx.x; e < 32 * 32; e += blockDim.x) {
        const int i = e >> 5, o = e & 31;
        const float v = (i < l1 && o < l2) ? l2_w[i * l2 + o] : 0.f;
        sw2[i][o] = v;
        sw2t[o][i] = v;
    }
    if (threadIdx.x < 32) {
        sb2[threadIdx.x] = (int)threadIdx.x < l2 ? l2_b[threadIdx.x] : 0.f;
        sw3[threadIdx.x] = (int)threadIdx.x < l2 ? l3_w[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const unsigned full = 0xffffffffu;
    const float b3 = l3_b[0];
    double e2 = 0.0;
    for (int b = blockIdx.x * wpb + (threadIdx.x >> 5); b < B; b += gridDim.x * wpb) {
        const float x1 = lane < l1 ? l1_pre[(size_t)b * l1 + lane] : 0.f;
        const float a1 = lane < l1 ? act_fwd(act, x1) : 0.f;
        float x2 = sb2[lane];
        for (int i = 0; i < l1; ++i) x2 += __shfl_sync(full, a1, i) * sw2[i][lane];
        const float a2 = lane < l2 ? act_fwd(act, x2) : 0.f;
        float part = a2 * sw3[lane];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(full, part, d);
        const float out = b3 + part;
        float dyv;
        const double contrib = loss_point(lp, out, score[b], wdl[b], &dyv);
        if (lane == 0) {
            e2 += contrib;
            net_output[b] = out;
            dy_out[b] = dyv;
        }
        if (backward) {
            const float d2 = lane < l2 ? act_grad(act, x2, dyv * sw3[lane]) : 0.f;
            float sum = 0.f;
            for (int o = 0; o < l2; ++o) sum += __shfl_sync(full, d2, o) * sw2t[o][lane];
            if (lane < l1) {
                dl1_pre[(size_t)b * l1 + lane] = act_grad(act, x1, sum);
                l1_acted_o[(size_t)b * l1 + lane] = a1;
            }
            if (lane < l2) {
                dl2_pre_o[(size_t)b * l2 + lane] = d2;
                l2_acted_o[(size_t)b * l2 + lane] = a2;
            }
        }
    }
    block_loss_partial(e2, loss_partials);
}

int launch_tail_simple(cudaStream_t s, const float* l1_pre, const float* score, const float* wdl,
                       const float* l2_w, const float* l2_b, const float* l3_w, const float* l3_b, LossParams lp,
                       int act, int B, int l1, int l2, float* net_output, float* dy, float* dl1_pre,
                       float* l1_acted, float* dl2_pre, float* l2_acted, double* loss_partials,
                       double* loss_acc, int backward) {
    const size_t smem = sizeof(float) * ((size_t)l1 * l2 + 2 * (size_t)l2);
    if (l1 <= 32 && l2 <= 32) {
        int blocks = ceil_div(B, 8);
        if (blocks > 148 * 4) blocks = 148 * 4;
        k_tail_simple_warp<<<blocks, 256, 0, s>>>(l1_pre, score, wdl, l2_w, l2_b, l3_w, l3_b, lp, act, B, l1, l2, net_output, dy,
                                                 dl1_pre, l1_acted, dl2_pre, l2_acted, loss_partials, backward);
        k_reduce_double<<<1, 256, 0, s>>>(loss_partials, blocks, loss_acc);
        return 2;
    }
    const int blocks = ceil_div(B, 128);
    k_tail_simple<<<blocks, 128, smem, s>>>(l1_pre, score, wdl, l2_w, l2_b, l3_w, l3_b, lp, act, B, l1, l2, net_output, dy,
                                           dl1_pre, l1_acted, dl2_pre, l2_acted, loss_partials, backward);
    k_reduce_double<<<1, 256, 0, s>>>(loss_partials, blocks, loss_acc);
    return 2;
}

// ------------------------------------------------------------------------------------------------
// Weight gradients of the small layers (L2, L3, their biases and the L1 biases), per bucket segment.
// cells of a segment: [0, R*C): sum_b U[b][cell / C] * V[b][cell % C]      (L2 weight)
//                     then l2: sum_b Bsrc[b][o]                           (L2 bias)
//                     then l2: sum_b l2_acted[b][o] * dy[b]               (L3 weight)
//                     then 1 : sum_b dy[b]                                (L3 bias)
//                     then l1: sum_b dl1[b][o]                            (L1 bias)
// grid (segments, SPLIT): block (g, s) reduces the s-th slice of segment g into partials; a second
// kernel adds the SPLIT partials in order.  No atomics: results do not depend on scheduling.
// (dense_mm_bucket.rs:112-161; native_kernels.cu:2591-2744 use register accumulators + atomics.)
// ------------------------------------------------------------------------------------------------
#define SW_CMAX 5
#define SW_SPLIT_LS 64  // blocks per bucket segment (LayerStack; 59, two exact waves, measured slower); the Simple net splits
                        // its one segment in 128
__global__ void __launch_bounds__(1024) k_small_wgrad(const int* __restrict__ order, const int* __restrict__ seg_start,
                                                       const float* __restrict__ U, int dimU, const float* __restrict__ V,
                                                       int dimV, const float* __restrict__ Bsrc, const float* __restrict__ l2_acted,
                                                       int l2, const float* __restrict__ dy, const float* __restrict__ dl1,
                                                       int l1, float* __restrict__ partials, int n_cells) {
    extern __shared__ float s_stage[];
    const int g = blockIdx.x, sp = blockIdx.y;
    const int SW_SPLIT = gridDim.y;
    const int sbeg = seg_start[g], send = seg_start[g + 1];
    const int len = send - sbeg;
    const int per = (len + SW_SPLIT - 1) / SW_SPLIT;
    const int beg = sbeg + min(sp * per, len), end = sbeg + min((sp + 1) * per, len);
    float* sU = s_stage;              // [32][dimU]
    float* sV = sU + 32 * dimU;       // [32][dimV]
    float* sB = sV + 32 * dimV;       // [32][l2]
    float* sA = sB + 32 * l2;         // [32][l2]
    float* sD = sA + 32 * l2;         // [32][l1]
    float* sY = sD + 32 * l1;         // [32]
    __shared__ int s_pos[32];
    const int nW = dimU * dimV;
    float acc[SW_CMAX];
#pragma unroll
    for (int j = 0; j < SW_CMAX; ++j) acc[j] = 0.f;
    for (int r0 = beg; r0 < end; r0 += 32) {
        const int cnt = min(32, end - r0);
        __syncthreads();
        if (threadIdx.x < 32) s_pos[threadIdx.x] = (int)threadIdx.x < cnt ? (order ? order[r0 + threadIdx.x] : r0 + threadIdx.x) : -1;
        __syncthreads();
        for (int e = threadIdx.x; e < 32 * dimU; e += blockDim.x) { const int r = e / dimU, c = e - r * dimU; const int p = s_pos[r]; sU[e] = p >= 0 ? U[(size_t)p * dimU + c] : 0.f; }
        for (int e = threadIdx.x; e < 32 * dimV; e += blockDim.x) { const int r = e / dimV, c = e - r * dimV; const int p = s_pos[r]; sV[e] = p >= 0 ? V[(size_t)p * dimV + c] : 0.f; }
        for (int e = threadIdx.x; e < 32 * l2; e += blockDim.x) {
            const int r = e / l2, c = e - r * l2; const int p = s_pos[r];
            sB[e] = p >= 0 ? Bsrc[(size_t)p * l2 + c] : 0.f;
            sA[e] = p >= 0 ? l2_acted[(size_t)p * l2 + c] : 0.f;
        }
        for (int e = threadIdx.x; e < 32 * l1; e += blockDim.x) { const int r = e / l1, c = e - r * l1; const int p = s_pos[r]; sD[e] = p >= 0 ? dl1[(size_t)p * l1 + c] : 0.f; }
        if (threadIdx.x < 32) { const int p = s_pos[threadIdx.x]; sY[threadIdx.x] = p >= 0 ? dy[p] : 0.f; }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < SW_CMAX; ++j) {
            const int cell = threadIdx.x + j * 1024;
            if (cell >= n_cells) continue;
            float a = acc[j];
            if (cell < nW) {
                const int u = cell / dimV, v = cell - u * dimV;
                for (int r = 0; r < cnt; ++r) a += sU[r * dimU + u] * sV[r * dimV + v];
            } else if (cell < nW + l2) {
                const int o = cell - nW;
                for (int r = 0; r < cnt; ++r) a += sB[r * l2 + o];
            } else if (cell < nW + 2 * l2) {
                const int o = cell - nW - l2;
                for (int r = 0; r < cnt; ++r) a += sA[r * l2 + o] * sY[r];
            } else if (cell == nW + 2 * l2) {
                for (int r = 0; r < cnt; ++r) a += sY[r];
            } else {
                const int o = cell - nW - 2 * l2 - 1;
                for (int r = 0; r < cnt; ++r) a += sD[r * l1 + o];
            }
            acc[j] = a;
        }
    }
#pragma unroll
    for (int j = 0; j < SW_CMAX; ++j) {
        const int cell = threadIdx.x + j * 1024;
        if (cell < n_cells) partials[((size_t)g * SW_SPLIT + sp) * n_cells + cell] = acc[j];
    }
}

// n_seg segments (the last one holds positions with an out-of-range bucket when has_invalid).  A warp per output
// cell: the lanes add the SW_SPLIT partials of the cell (lane l takes l, l + 32, ...), then a shuffle tree; a fixed order.
static __device__ __forceinline__ float sw_cell_sum(const float* __restrict__ partials, int g, int SW_SPLIT, int n_cells, int cell,
                                                    int lane) {
    float sum = 0.f;
    for (int sp = lane; sp < SW_SPLIT; sp += 32) sum += partials[((size_t)g * SW_SPLIT + sp) * n_cells + cell];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    return sum;
}

__global__ void __launch_bounds__(256) k_small_wgrad_final(const float* __restrict__ partials, int n_seg, int has_invalid, int SW_SPLIT,
                                                            int n_cells, int nW, int l2, int l1, float* __restrict__ gw2,
                                                            float* __restrict__ gb2, float* __restrict__ gw3, float* __restrict__ gb3,
                                                            float* __restrict__ gb1, float* __restrict__ gb1_shared) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // warp index
    const int n_real = has_invalid ? n_seg - 1 : n_seg;
    if (i < n_real * n_cells) {
        const int g = i / n_cells, cell = i - g * n_cells;
        const float sum = sw_cell_sum(partials, g, SW_SPLIT, n_cells, cell, lane);
        if (lane == 0) {
            if (cell < nW) gw2[(size_t)g * nW + cell] = sum;
            else if (cell < nW + l2) gb2[g * l2 + (cell - nW)] = sum;
            else if (cell < nW + 2 * l2) gw3[g * l2 + (cell - nW - l2)] = sum;
            else if (cell == nW + 2 * l2) gb3[g] = sum;
            else gb1[g * l1 + (cell - nW - 2 * l2 - 1)] = sum;
        }
    } else if (gb1_shared && i < n_real * n_cells + l1) {
        // shared L1 bias: every position contributes, also those with an out-of-range bucket
        const int cell = nW + 2 * l2 + 1 + (i - n_real * n_cells);
        float tot = 0.f;
        for (int g = 0; g < n_seg; ++g) tot += sw_cell_sum(partials, g, SW_SPLIT, n_cells, cell, lane);
        if (lane == 0) gb1_shared[i - n_real * n_cells] = tot;
    }
}

static int small_wgrad(cudaStream_t s, const int* order, const int* seg_start, int n_seg, int has_invalid, int split,
                       const float* U, int dimU, const float* V, int dimV, const float* Bsrc, const float* l2_acted,
                       int l2, const float* dy, const float* dl1, int l1, float* partials, float* gw2, float* gb2,
                       float* gw3, float* gb3, float* gb1, float* gb1_shared) {
    const int nW = dimU * dimV;
    const int n_cells = nW + 2 * l2 + 1 + l1;
    const size_t smem = sizeof(float) * 32 * ((size_t)dimU + dimV + 2 * l2 + l1 + 1);
    cudaFuncSetAttribute(k_small_wgrad, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    k_small_wgrad<<<dim3(n_seg, split), 1024, smem, s>>>(order, seg_start, U, dimU, V, dimV, Bsrc, l2_acted, l2, dy, dl1,
                                                          l1, partials, n_cells);
    const int n = n_seg * n_cells + l1;  // warps
    k_small_wgrad_final<<<ceil_div(n, 8), 256, 0, s>>>(partials, n_seg, has_invalid, split, n_cells, nW, l2, l1, gw2,
                                                                      gb2, gw3, gb3, gb1, gb1_shared);
    return 2;
}

int launch_small_wgrad_layerstack(cudaStream_t s, const int* order, const int* seg_start, int B, int l1, int l2,
                                  int nb, const float* l2_input, const float* dl2_out, const float* l2_acted,
                                  const float* dy, const float* dl1_total, float* partials, float* l2_w_grad,
                                  float* l2_b_grad, float* l3_w_grad, float* l3_b_grad, float* l1_b_grad,
                                  float* l1s_b_grad) {
    (void)B;
    // L2 weight cell (o, i) = sum dl2_out[b][o] * l2_input[b][i]
    return small_wgrad(s, order, seg_start, nb + 1, 1, SW_SPLIT_LS, dl2_out, l2, l2_input, 2 * (l1 - 1), dl2_out, l2_acted, l2, dy,
                       dl1_total, l1, partials, l2_w_grad, l2_b_grad, l3_w_grad, l3_b_grad, l1_b_grad, l1s_b_grad);
}

int launch_small_wgrad_simple(cudaStream_t s, const int* order, const int* seg_start, int B, int l1, int l2,
                              const float* l1_acted, const float* dl2_pre, const float* l2_acted, const float* dy,
                              const float* dl1_pre, float* partials, float* l2_w_grad, float* l2_b_grad,
                              float* l3_w_grad, float* l3_b_grad, float* l1_b_grad) {
    (void)B;
    // L2 weight cell (i, o) = sum l1_acted[b][i] * dl2_pre[b][o]; the whole batch is one segment
    return small_wgrad(s, order, seg_start, 1, 0, 128, l1_acted, l1, dl2_pre, l2, dl2_pre, l2_acted, l2, dy, dl1_pre, l1,
                       partials, l2_w_grad, l2_b_grad, l3_w_grad, l3_b_grad, l1_b_grad, nullptr);
}

// ------------------------------------------------------------------------------------------------
// L1 weight gradient.  gw_bucket[g][o][k] = sum over positions of bucket g of dl1[b][o] * x[b][k]
// (dense_mm_bucket.rs:112-135); gw_shared[k][o] = the same sum over every position (dense_mm.rs:75-92),
// obtained as the sum of the per-bucket results.  Work unit = up to TB_UNIT_TILES tiles of one bucket;
// block (column chunk of 128, unit) writes partials[unit][o][k]; the second kernel adds the units of
// each bucket in order.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_l1_wgrad(const float* __restrict__ x, int K, const float* __restrict__ dl1,
                                                   const int* __restrict__ order, const TileDesc* __restrict__ tiles,
                                                   const TileDesc* __restrict__ units, const int* __restrict__ n_units, int l1,
                                                   float* __restrict__ partials) {
    const int u = blockIdx.y;
    if (u >= *n_units) return;
    const TileDesc ud = units[u];
    __shared__ float sdl[TB_TILE_M][TB_MAX_L1];
    __shared__ int s_pos[TB_TILE_M];
    const int col = blockIdx.x * 128 + (threadIdx.x & 127);
    const int oh = threadIdx.x >> 7;
    float acc[TB_MAX_L1 / 2];
#pragma unroll
    for (int j = 0; j < TB_MAX_L1 / 2; ++j) acc[j] = 0.f;
    for (int t = ud.start; t < ud.start + ud.count; ++t) {
        const TileDesc td = tiles[t];
        __syncthreads();
        if (threadIdx.x < TB_TILE_M) s_pos[threadIdx.x] = (int)threadIdx.x < td.count ? order[td.start + threadIdx.x] : -1;
        __syncthreads();
        for (int e = threadIdx.x; e < TB_TILE_M * l1; e += 256) {
            const int r = e / l1, o = e - r * l1;
            const int p = s_pos[r];
            sdl[r][o] = p >= 0 ? dl1[(size_t)p * l1 + o] : 0.f;
        }
        __syncthreads();
        for (int r0 = 0; r0 < td.count; r0 += 4) {
            float xv[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int p = r0 + q < td.count ? s_pos[r0 + q] : -1;
                xv[q] = p >= 0 ? __ldg(x + (size_t)p * K + col) : 0.f;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (r0 + q < td.count) {
#pragma unroll
                    for (int j = 0; j < TB_MAX_L1 / 2; ++j) {
                        const int o = oh + 2 * j;
                        if (o < l1) acc[j] += sdl[r0 + q][o] * xv[q];
                    }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < TB_MAX_L1 / 2; ++j) {
        const int o = oh + 2 * j;
        if (o < l1) partials[((size_t)u * l1 + o) * K + col] = acc[j];
    }
}

// Second stage: block column g adds the work units of bucket g in order (the units of a bucket are contiguous);
// the last column (g == nb: positions with an out-of-range bucket id, or the whole batch for Simple) goes to a
// scratch row.  Third stage: gw_shared[k][o] = sum over the columns.
__global__ void __launch_bounds__(256) k_l1_wgrad_final(const float* __restrict__ partials, const TileDesc* __restrict__ units,
                                                         const int* __restrict__ n_units, int K, int l1, int nb,
                                                         float* __restrict__ gw_bucket, float* __restrict__ rest) {
    __shared__ int s_range[2];
    const int g = blockIdx.y;
    const int nu = *n_units;
    if (threadIdx.x == 0) { s_range[0] = nu; s_range[1] = nu; }
    __syncthreads();
    for (int u = threadIdx.x; u < nu; u += blockDim.x) {  // first unit of bucket g, first unit of a later bucket
        const int bk = units[u].bucket;
        if (bk == g) atomicMin(&s_range[0], u);
        if (bk > g) atomicMin(&s_range[1], u);
    }
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= l1 * K) return;
    const int u0 = s_range[0], u1 = s_range[1];
    float sum = 0.f;
    int u = u0;
    for (; u + 4 <= u1; u += 4) {  // four loads in flight, added in unit order
        const float a = partials[(size_t)u * l1 * K + i], b = partials[(size_t)(u + 1) * l1 * K + i];
        const float c = partials[(size_t)(u + 2) * l1 * K + i], d = partials[(size_t)(u + 3) * l1 * K + i];
        sum += a; sum += b; sum += c; sum += d;
    }
    for (; u < u1; ++u) sum += partials[(size_t)u * l1 * K + i];
    if (g < nb) gw_bucket[(size_t)g * l1 * K + i] = sum;
    else rest[i] = sum;
}

__global__ void __launch_bounds__(256) k_l1_wgrad_shared(const float* __restrict__ gw_bucket, const float* __restrict__ rest,
                                                          int K, int l1, int nb, float* __restrict__ gw_shared) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= l1 * K) return;
    const int o = i / K, k = i - o * K;
    float total = 0.f;
    for (int g = 0; g < nb; ++g) total += gw_bucket[(size_t)g * l1 * K + i];
    total += rest[i];
    gw_shared[(size_t)k * l1 + o] = total;
}

// Variant for l1 % 8 == 0: a thread owns four adjacent columns and OPT outputs (OPT = 8 or 16; two thread groups
// split the outputs when l1 = 32), so that one 128-bit load of x feeds 4 * OPT multiply-adds and the dl1 values
// come as broadcast 128-bit shared-memory loads.  The unit's positions (consecutive in the bucket order) and their dl1
// rows are staged once, then the x rows arrive through a private ring of asynchronous copies (a thread copies the 16
// bytes it reads itself), WG_STAGES rounds of four positions ahead of the arithmetic.
#define WG_POS (TB_UNIT_TILES * TB_TILE_M)
#define WG_STAGES 2
template <int OPT, int THREADS, int MIN_BLOCKS>
__global__ void __launch_bounds__(THREADS, MIN_BLOCKS) k_l1_wgrad_stream(const float* __restrict__ x, int K, const float* __restrict__ dl1,
                                                          const int* __restrict__ order, const TileDesc* __restrict__ tiles,
                                                          const TileDesc* __restrict__ units, const int* __restrict__ n_units, int l1,
                                                          float* __restrict__ partials) {
    extern __shared__ __align__(16) unsigned char s_dyn[];  // sdl [WG_POS][l1] floats, then the ring [WG_STAGES][4][threads] float4
    __shared__ int s_pos[WG_POS];
    const int u = blockIdx.y;
    if (u >= *n_units) return;
    const TileDesc ud = units[u];
    const int K4 = K >> 2;
    const int tcol = threadIdx.x & 127, og = threadIdx.x >> 7;
    const int col4 = min(blockIdx.x * 128 + tcol, K4 - 1);  // a thread past the last column repeats it and drops its result
    const bool active = blockIdx.x * 128 + tcol < K4;
    const int p_begin = tiles[ud.start].start;
    const TileDesc tl = tiles[ud.start + ud.count - 1];
    const int n = tl.start + tl.count - p_begin;
    float* sdl = reinterpret_cast<float*>(s_dyn);
    float4* ring = reinterpret_cast<float4*>(s_dyn + (size_t)WG_POS * l1 * sizeof(float));
    for (int i = threadIdx.x; i < WG_POS; i += blockDim.x) s_pos[i] = i < n ? order[p_begin + i] : -1;
    __syncthreads();
    const int l1q = l1 >> 2;
    for (int e = threadIdx.x; e < n * l1q; e += blockDim.x) {
        const int r = e / l1q, o4 = e - r * l1q;
        reinterpret_cast<float4*>(sdl + (size_t)r * l1)[o4] = *reinterpret_cast<const float4*>(dl1 + (size_t)s_pos[r] * l1 + 4 * o4);
    }
    const int T = blockDim.x;
    const float4* __restrict__ x4 = reinterpret_cast<const float4*>(x);
    auto issue = [&](int round) {
        if (4 * round < n) {
            const int stage = round % WG_STAGES;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = 4 * round + q;
                dg_cp16(ring + (size_t)(stage * 4 + q) * T + threadIdx.x, x4 + (size_t)s_pos[r < n ? r : 0] * K4 + col4);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float4 acc[OPT];
#pragma unroll
    for (int j = 0; j < OPT; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int n_rounds = (n + 3) >> 2;
#pragma unroll
    for (int r = 0; r < WG_STAGES - 1; ++r) issue(r);
    __syncthreads();  // dl1 rows staged
    for (int round = 0; round < n_rounds; ++round) {
        issue(round + WG_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(WG_STAGES - 1) : "memory");
        const int stage = round % WG_STAGES;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int r = 4 * round + q;
            if (r >= n) break;
            const float4 xv = ring[(size_t)(stage * 4 + q) * T + threadIdx.x];
#pragma unroll
            for (int j4 = 0; j4 < OPT / 4; ++j4) {
                const float4 g = *reinterpret_cast<const float4*>(sdl + (size_t)r * l1 + og * OPT + 4 * j4);
                const float gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[4 * j4 + j].x += gv[j] * xv.x;
                    acc[4 * j4 + j].y += gv[j] * xv.y;
                    acc[4 * j4 + j].z += gv[j] * xv.z;
                    acc[4 * j4 + j].w += gv[j] * xv.w;
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (!active) return;
#pragma unroll
    for (int j = 0; j < OPT; ++j) {
        const int o = og * OPT + j;
        reinterpret_cast<float4*>(partials + ((size_t)u * l1 + o) * K)[col4] = acc[j];
    }
}

int launch_l1_wgrad(cudaStream_t s, const float* x, int K, const float* dl1, const int* order,
                    const TileDesc* tiles, const int* n_tiles, int max_tiles, int l1, int nb, float* partials,
                    float* gw_bucket, float* gw_shared) {
    const TileDesc* units = tiles + max_tiles;
    const int* n_units = n_tiles + 1;
    const int max_units = sort_max_units(max_tiles);
    if (l1 == 8 || l1 == 16 || l1 == 32) {
        const int threads = l1 == 32 ? 256 : 128;
        const size_t smem = (size_t)WG_POS * l1 * sizeof(float) + (size_t)WG_STAGES * 4 * threads * 16;
        const dim3 grid(ceil_div(K / 4, 128), max_units);
        // 128-thread blocks at six per SM: with K = 1536 the 3 x 265 blocks of the benchmark then run as one wave
        if (l1 == 8) {
            cudaFuncSetAttribute(k_l1_wgrad_stream<8, 128, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            k_l1_wgrad_stream<8, 128, 6><<<grid, threads, smem, s>>>(x, K, dl1, order, tiles, units, n_units, l1, partials);
        } else if (l1 == 16) {
            cudaFuncSetAttribute(k_l1_wgrad_stream<16, 128, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            k_l1_wgrad_stream<16, 128, 6><<<grid, threads, smem, s>>>(x, K, dl1, order, tiles, units, n_units, l1, partials);
        } else {
            cudaFuncSetAttribute(k_l1_wgrad_stream<16, 256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            k_l1_wgrad_stream<16, 256, 2><<<grid, threads, smem, s>>>(x, K, dl1, order, tiles, units, n_units, l1, partials);
        }
    } else
        k_l1_wgrad<<<dim3(K / 128, max_units), 256, 0, s>>>(x, K, dl1, order, tiles, units, n_units, l1, partials);
    float* rest = partials + (size_t)max_units * l1 * K;  // one more [l1][K] row behind the unit partials
    k_l1_wgrad_final<<<dim3(ceil_div(l1 * K, 256), nb + 1), 256, 0, s>>>(partials, units, n_units, K, l1, nb, gw_bucket, rest);
    k_l1_wgrad_shared<<<ceil_div(l1 * K, 256), 256, 0, s>>>(gw_bucket, rest, K, l1, nb, gw_shared);
    return 3;
}

// ------------------------------------------------------------------------------------------------
// L1 input gradient fused with the FT activation gradient.
//   d[b, c] = sum_o dl1[b, o] * (wb[g, o, c] + ws[c, o])          (never written to memory)
// LayerStack (mode 1): c = persp*F/2 + r is the pair (r, r + F/2) of one perspective,
//   dft[b, r]       = 0 < xa < 1 ? d * crelu(xb) * scale : 0      xa = pre[b, r] + bias[r]
//   dft[b, r + F/2] = 0 < xb < 1 ? d * crelu(xa) * scale : 0      xb = pre[b, r + F/2] + bias[r + F/2]
//   (ft_post_perspective.rs:92-129 on the sum of the two L1 input gradients, native_kernels.cu:2260)
// Simple (mode 2 CReLU / 3 SCReLU): c = persp*F + col, pre already holds the biased value,
//   dft[b, col] = act'(pre[b, col]) * d                            (native_kernels.cu:1452-1497)
// The FT bias gradient is accumulated per block in registers and written as one partial row per block.
// grid (n_ctas, 2 perspectives, column chunks); a block walks the tiles t = blockIdx.x, += gridDim.x and
// keeps the effective weights of the current bucket in shared memory.
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(256) k_l1_dgrad_ftgrad(const float* __restrict__ dl1, const int* __restrict__ order,
                                                          const TileDesc* __restrict__ tiles, const int* __restrict__ n_tiles,
                                                          const float* __restrict__ wb, const float* __restrict__ ws,
                                                          const float* __restrict__ pre_stm, const float* __restrict__ pre_nstm,
                                                          const float* __restrict__ ft_bias, float scale, int F, int l1, int nb,
                                                          int CW, float* __restrict__ dft_stm, float* __restrict__ dft_nstm,
                                                          float* __restrict__ bias_partials) {
    extern __shared__ float s_weff[];  // [l1][CW]
    __shared__ float sdl[TB_TILE_M][TB_MAX_L1];
    __shared__ int s_pos[TB_TILE_M];
    const int persp = blockIdx.y;
    const int chunk = blockIdx.z;
    const int half = F >> 1;
    const int Kin = MODE == 1 ? F : 2 * F;                        // row length of the L1 input
    const int cbase = (MODE == 1 ? persp * half : persp * F) + chunk * CW;  // first L1 input column of this block
    const int wcol = chunk * CW + 4 * threadIdx.x;                // column inside the perspective
    const float* __restrict__ pre = persp ? pre_nstm : pre_stm;
    float* __restrict__ dft = persp ? dft_nstm : dft_stm;
    const int nt = *n_tiles;
    int cur_bucket = -1;
    float4 bacc0 = make_float4(0.f, 0.f, 0.f, 0.f), bacc1 = bacc0;
    float4 bias0 = make_float4(0.f, 0.f, 0.f, 0.f), bias1 = bias0;
    if (MODE == 1) {
        bias0 = *reinterpret_cast<const float4*>(ft_bias + wcol);
        bias1 = *reinterpret_cast<const float4*>(ft_bias + half + wcol);
    }
    for (int t = blockIdx.x; t < nt; t += gridDim.x) {
        const TileDesc td = tiles[t];
        __syncthreads();
        if (td.bucket != cur_bucket) {
            cur_bucket = td.bucket;
            const bool use_b = wb != nullptr && td.bucket < nb;
            for (int e = threadIdx.x; e < l1 * CW; e += blockDim.x) {
                const int o = e / CW, c = e - o * CW;
                float v = ws[(size_t)(cbase + c) * l1 + o];
                if (use_b) v = wb[((size_t)td.bucket * l1 + o) * Kin + cbase + c] + v;
                s_weff[e] = v;
            }
        }
        for (int i = threadIdx.x; i < TB_TILE_M; i += blockDim.x) s_pos[i] = i < td.count ? order[td.start + i] : -1;
        __syncthreads();
        for (int e = threadIdx.x; e < TB_TILE_M * l1; e += blockDim.x) {
            const int r = e / l1, o = e - r * l1;
            const int p = s_pos[r];
            sdl[r][o] = p >= 0 ? dl1[(size_t)p * l1 + o] : 0.f;
        }
        __syncthreads();
        for (int r0 = 0; r0 < td.count; r0 += 2) {
            float4 xa[2], xb[2];
            int pp[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                pp[q] = r0 + q < td.count ? s_pos[r0 + q] : -1;
                if (pp[q] >= 0) {
                    xa[q] = *reinterpret_cast<const float4*>(pre + (size_t)pp[q] * F + wcol);
                    if (MODE == 1) xb[q] = *reinterpret_cast<const float4*>(pre + (size_t)pp[q] * F + half + wcol);
                }
            }
            float4 dd[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
            for (int o = 0; o < l1; ++o) {
                const float4 w4 = *reinterpret_cast<const float4*>(s_weff + o * CW + 4 * threadIdx.x);
                const float g0 = sdl[r0][o], g1 = sdl[r0 + 1 < TB_TILE_M ? r0 + 1 : r0][o];
                dd[0].x += g0 * w4.x; dd[0].y += g0 * w4.y; dd[0].z += g0 * w4.z; dd[0].w += g0 * w4.w;
                dd[1].x += g1 * w4.x; dd[1].y += g1 * w4.y; dd[1].z += g1 * w4.z; dd[1].w += g1 * w4.w;
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                if (pp[q] < 0) continue;
                const float4 d = dd[q];
                if (MODE == 1) {
                    const float4 a = make_float4(xa[q].x + bias0.x, xa[q].y + bias0.y, xa[q].z + bias0.z, xa[q].w + bias0.w);
                    const float4 b = make_float4(xb[q].x + bias1.x, xb[q].y + bias1.y, xb[q].z + bias1.z, xb[q].w + bias1.w);
                    float4 ga, gb;
                    ga.x = (a.x > 0.f && a.x < 1.f) ? d.x * crelu01(b.x) * scale : 0.f;
                    ga.y = (a.y > 0.f && a.y < 1.f) ? d.y * crelu01(b.y) * scale : 0.f;
                    ga.z = (a.z > 0.f && a.z < 1.f) ? d.z * crelu01(b.z) * scale : 0.f;
                    ga.w = (a.w > 0.f && a.w < 1.f) ? d.w * crelu01(b.w) * scale : 0.f;
                    gb.x = (b.x > 0.f && b.x < 1.f) ? d.x * crelu01(a.x) * scale : 0.f;
                    gb.y = (b.y > 0.f && b.y < 1.f) ? d.y * crelu01(a.y) * scale : 0.f;
                    gb.z = (b.z > 0.f && b.z < 1.f) ? d.z * crelu01(a.z) * scale : 0.f;
                    gb.w = (b.w > 0.f && b.w < 1.f) ? d.w * crelu01(a.w) * scale : 0.f;
                    *reinterpret_cast<float4*>(dft + (size_t)pp[q] * F + wcol) = ga;   // re-read 40 times by the FT backward: keep in L2
                    *reinterpret_cast<float4*>(dft + (size_t)pp[q] * F + half + wcol) = gb;
                    bacc0.x += ga.x; bacc0.y += ga.y; bacc0.z += ga.z; bacc0.w += ga.w;
                    bacc1.x += gb.x; bacc1.y += gb.y; bacc1.z += gb.z; bacc1.w += gb.w;
                } else {
                    const float4 x = xa[q];
                    float4 g;
                    if (MODE == 2) {
                        g.x = (x.x > 0.f && x.x < 1.f) ? d.x : 0.f;
                        g.y = (x.y > 0.f && x.y < 1.f) ? d.y : 0.f;
                        g.z = (x.z > 0.f && x.z < 1.f) ? d.z : 0.f;
                        g.w = (x.w > 0.f && x.w < 1.f) ? d.w : 0.f;
                    } else {
                        const float4 a = make_float4(crelu01(x.x), crelu01(x.y), crelu01(x.z), crelu01(x.w));
                        g.x = d.x * ((a.x > 0.f && a.x < 1.f) ? 2.0f * a.x : 0.f);
                        g.y = d.y * ((a.y > 0.f && a.y < 1.f) ? 2.0f * a.y : 0.f);
                        g.z = d.z * ((a.z > 0.f && a.z < 1.f) ? 2.0f * a.z : 0.f);
                        g.w = d.w * ((a.w > 0.f && a.w < 1.f) ? 2.0f * a.w : 0.f);
                    }
                    *reinterpret_cast<float4*>(dft + (size_t)pp[q] * F + wcol) = g;
                    bacc0.x += g.x; bacc0.y += g.y; bacc0.z += g.z; bacc0.w += g.w;
                }
            }
        }
    }
    // one partial row per (block, perspective): [n_ctas][2][F]
    float* bp = bias_partials + ((size_t)blockIdx.x * 2 + persp) * F;
    *reinterpret_cast<float4*>(bp + wcol) = bacc0;
    if (MODE == 1) *reinterpret_cast<float4*>(bp + half + wcol) = bacc1;
}

// Streaming variant for l1 = 8, 16 or 32.  A thread keeps the effective weights of its four columns ([L1] float4) in
// registers, so a position costs L1 / 4 broadcast loads of its dl1 row from shared memory and 4 * L1 multiply-adds:
// the shared-memory pipe is not the limit.  A block owns half a work unit (<= DG_POS consecutive positions of the
// bucket order, one bucket) and one perspective; the pre-activations arrive through a private ring of asynchronous
// copies (every thread copies exactly the 16-byte pieces it reads itself, so no barrier is needed), DG_STAGES rounds
// of four positions ahead of the arithmetic, which keeps the global loads in flight back to back.
#define DG_POS 128     // positions per block
#define DG_STAGES 3
static_assert(2 * DG_POS == TB_UNIT_TILES * TB_TILE_M, "a block of the streaming kernel owns half a work unit");
// HALF: pre-activations and dft rows are fp16 (ft_post_perspective_grad_fused_fp16, native_kernels.cu:2304-2353): the
// gradient is multiplied by grad_scale, clamped to the fp16 range (clamps are counted) and rounded; the bias gradient
// takes the unscaled fp32 value.
template <int MODE, int L1, bool HALF>
__global__ void __launch_bounds__(256) k_l1_dgrad_ftgrad_stream(const float* __restrict__ dl1, const int* __restrict__ order,
                                                                 const TileDesc* __restrict__ tiles, const TileDesc* __restrict__ units,
                                                                 const int* __restrict__ n_units, const float* __restrict__ wb,
                                                                 const float* __restrict__ ws, const void* __restrict__ pre_stm,
                                                                 const void* __restrict__ pre_nstm, const float* __restrict__ ft_bias,
                                                                 float scale, int F, int nb, int CW, void* __restrict__ dft_stm,
                                                                 void* __restrict__ dft_nstm, float* __restrict__ bias_partials,
                                                                 float grad_scale, unsigned long long* __restrict__ clamp_counter) {
    constexpr int NP = MODE == 1 ? 2 : 1;  // pieces per position and thread
    constexpr int ESZ = HALF ? 2 : 4;      // bytes per pre-activation / dft element
    typedef typename std::conditional<HALF, uint2, float4>::type Piece;  // a thread's four columns of one row
    extern __shared__ __align__(16) unsigned char s_dyn[];  // ring [DG_STAGES][4 positions][NP][threads] pieces
    __shared__ __align__(16) float sdl[DG_POS][L1];
    __shared__ int s_pos[DG_POS];
    const int persp = blockIdx.y;
    const int chunk = blockIdx.z;
    const int half = F >> 1;
    const int Kin = MODE == 1 ? F : 2 * F;                        // row length of the L1 input
    const int cbase = (MODE == 1 ? persp * half : persp * F) + chunk * CW;  // first L1 input column of this block
    const int wcol = chunk * CW + 4 * threadIdx.x;                // column inside the perspective
    const unsigned char* __restrict__ pre = static_cast<const unsigned char*>(persp ? pre_nstm : pre_stm);
    unsigned char* __restrict__ dft = static_cast<unsigned char*>(persp ? dft_nstm : dft_stm);
    float4 bacc0 = make_float4(0.f, 0.f, 0.f, 0.f), bacc1 = bacc0;
    float* bp = bias_partials + ((size_t)blockIdx.x * 2 + persp) * F;  // one partial row per (block, perspective)
    unsigned clamps = 0;

    // the block's positions: tiles [first, last) of unit blockIdx.x / 2, contiguous in the bucket order
    const int u = blockIdx.x >> 1, h = blockIdx.x & 1;
    int p_begin = 0, n = 0, bucket = 0;
    if (u < *n_units) {
        const TileDesc ud = units[u];
        const int per = DG_POS / TB_TILE_M;
        const int first = ud.start + h * per, last = min(ud.start + ud.count, first + per);
        if (first < last) {
            p_begin = tiles[first].start;
            n = tiles[last - 1].start + tiles[last - 1].count - p_begin;
            bucket = ud.bucket;
        }
    }
    if (n == 0) {  // the bias reduction reads every row
        *reinterpret_cast<float4*>(bp + wcol) = bacc0;
        if (MODE == 1) *reinterpret_cast<float4*>(bp + half + wcol) = bacc1;
        return;
    }
    for (int i = threadIdx.x; i < DG_POS; i += blockDim.x) s_pos[i] = i < n ? order[p_begin + i] : -1;
    // effective weights of the thread's four columns
    float4 w[L1];
    {
        const bool use_b = wb != nullptr && bucket < nb;
        const int c0 = cbase + 4 * threadIdx.x;
#pragma unroll
        for (int o4 = 0; o4 < L1 / 4; ++o4) {
            const float4 r0 = *reinterpret_cast<const float4*>(ws + (size_t)(c0 + 0) * L1 + 4 * o4);
            const float4 r1 = *reinterpret_cast<const float4*>(ws + (size_t)(c0 + 1) * L1 + 4 * o4);
            const float4 r2 = *reinterpret_cast<const float4*>(ws + (size_t)(c0 + 2) * L1 + 4 * o4);
            const float4 r3 = *reinterpret_cast<const float4*>(ws + (size_t)(c0 + 3) * L1 + 4 * o4);
            w[4 * o4 + 0] = make_float4(r0.x, r1.x, r2.x, r3.x);
            w[4 * o4 + 1] = make_float4(r0.y, r1.y, r2.y, r3.y);
            w[4 * o4 + 2] = make_float4(r0.z, r1.z, r2.z, r3.z);
            w[4 * o4 + 3] = make_float4(r0.w, r1.w, r2.w, r3.w);
        }
        if (use_b) {
#pragma unroll
            for (int o = 0; o < L1; ++o) {
                const float4 v = *reinterpret_cast<const float4*>(wb + ((size_t)bucket * L1 + o) * Kin + c0);
                w[o].x = v.x + w[o].x; w[o].y = v.y + w[o].y; w[o].z = v.z + w[o].z; w[o].w = v.w + w[o].w;
            }
        }
    }
    float4 bias0 = make_float4(0.f, 0.f, 0.f, 0.f), bias1 = bias0;
    if (MODE == 1) {
        bias0 = *reinterpret_cast<const float4*>(ft_bias + wcol);
        bias1 = *reinterpret_cast<const float4*>(ft_bias + half + wcol);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < DG_POS * L1 / 4; e += blockDim.x) {
        const int r = e / (L1 / 4), o4 = e - r * (L1 / 4);
        const int p = s_pos[r];
        reinterpret_cast<float4*>(&sdl[r][0])[o4] = p >= 0 ? *reinterpret_cast<const float4*>(dl1 + (size_t)p * L1 + 4 * o4)
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // ring slot of (stage, position q, piece k) of this thread
    Piece* ring = reinterpret_cast<Piece*>(s_dyn);
    const int T = blockDim.x;
    auto slot = [&](int stage, int q, int k) { return ring + ((size_t)(stage * 4 + q) * NP + k) * T + threadIdx.x; };
    auto copy_piece = [&](Piece* dst, const unsigned char* src) { if (HALF) dg_cp8(dst, src); else dg_cp16(dst, src); };
    auto to_f4 = [&](const Piece& pc) {
        if constexpr (HALF) { const float2 a = dk_unpack_h2(pc.x), b = dk_unpack_h2(pc.y); return make_float4(a.x, a.y, b.x, b.y); }
        else return pc;
    };
    // stores a thread's four gradient values of one row: fp32 as they are; fp16 scaled, clamped, rounded
    auto store_dft = [&](unsigned char* dst, const float4& gv) {
        if constexpr (HALF) {
            float a = gv.x * grad_scale, b = gv.y * grad_scale, c = gv.z * grad_scale, d = gv.w * grad_scale;
            // one test for the four values; beyond the fp16 range (rare) each is clamped and counted.  A NaN passes the
            // test as it passes the reference's comparisons, and is stored as NaN.
            if (fmaxf(fmaxf(fabsf(a), fabsf(b)), fmaxf(fabsf(c), fabsf(d))) > 65504.0f) {
                a = clamp_half_count(a, clamps); b = clamp_half_count(b, clamps);
                c = clamp_half_count(c, clamps); d = clamp_half_count(d, clamps);
            }
            *reinterpret_cast<uint2*>(dst) = make_uint2(dk_pack_h2(a, b), dk_pack_h2(c, d));
        } else {
            *reinterpret_cast<float4*>(dst) = gv;
        }
    };
    auto issue = [&](int round) {  // copies of positions 4 * round .. + 3 (a missing position repeats the block's first)
        if (4 * round < n) {
            const int stage = round % DG_STAGES;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int r = 4 * round + q;
                const int pl = s_pos[r < n ? r : 0];
                copy_piece(slot(stage, q, 0), pre + ((size_t)pl * F + wcol) * ESZ);
                if (MODE == 1) copy_piece(slot(stage, q, 1), pre + ((size_t)pl * F + half + wcol) * ESZ);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per round, empty past the end
    };
    const int n_rounds = (n + 3) >> 2;
#pragma unroll
    for (int r = 0; r < DG_STAGES - 1; ++r) issue(r);
    __syncthreads();  // dl1 rows staged
    for (int round = 0; round < n_rounds; ++round) {
        issue(round + DG_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(DG_STAGES - 1) : "memory");  // this round's copies have landed
        const int stage = round % DG_STAGES;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int r = 4 * round + q;
            if (r >= n) break;
            const int pp = s_pos[r];
            float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4* gr = reinterpret_cast<const float4*>(&sdl[r][0]);
#pragma unroll
            for (int o4 = 0; o4 < L1 / 4; ++o4) {
                const float4 g = gr[o4];
                const float gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                for (int uu = 0; uu < 4; ++uu) {
                    const float4 ww = w[4 * o4 + uu];
                    d.x += gv[uu] * ww.x; d.y += gv[uu] * ww.y; d.z += gv[uu] * ww.z; d.w += gv[uu] * ww.w;
                }
            }
            const float4 xa = to_f4(*slot(stage, q, 0));
            if (MODE == 1) {
                const float4 xb = to_f4(*slot(stage, q, 1));
                const float4 a = make_float4(xa.x + bias0.x, xa.y + bias0.y, xa.z + bias0.z, xa.w + bias0.w);
                const float4 b = make_float4(xb.x + bias1.x, xb.y + bias1.y, xb.z + bias1.z, xb.w + bias1.w);
                float4 ga, gb;
                ga.x = (a.x > 0.f && a.x < 1.f) ? d.x * crelu01(b.x) * scale : 0.f;
                ga.y = (a.y > 0.f && a.y < 1.f) ? d.y * crelu01(b.y) * scale : 0.f;
                ga.z = (a.z > 0.f && a.z < 1.f) ? d.z * crelu01(b.z) * scale : 0.f;
                ga.w = (a.w > 0.f && a.w < 1.f) ? d.w * crelu01(b.w) * scale : 0.f;
                gb.x = (b.x > 0.f && b.x < 1.f) ? d.x * crelu01(a.x) * scale : 0.f;
                gb.y = (b.y > 0.f && b.y < 1.f) ? d.y * crelu01(a.y) * scale : 0.f;
                gb.z = (b.z > 0.f && b.z < 1.f) ? d.z * crelu01(a.z) * scale : 0.f;
                gb.w = (b.w > 0.f && b.w < 1.f) ? d.w * crelu01(a.w) * scale : 0.f;
                store_dft(dft + ((size_t)pp * F + wcol) * ESZ, ga);   // read again by the FT backward: keep in L2
                store_dft(dft + ((size_t)pp * F + half + wcol) * ESZ, gb);
                bacc0.x += ga.x; bacc0.y += ga.y; bacc0.z += ga.z; bacc0.w += ga.w;
                bacc1.x += gb.x; bacc1.y += gb.y; bacc1.z += gb.z; bacc1.w += gb.w;
            } else {
                const float4 x = xa;
                float4 g;
                if (MODE == 2) {
                    g.x = (x.x > 0.f && x.x < 1.f) ? d.x : 0.f;
                    g.y = (x.y > 0.f && x.y < 1.f) ? d.y : 0.f;
                    g.z = (x.z > 0.f && x.z < 1.f) ? d.z : 0.f;
                    g.w = (x.w > 0.f && x.w < 1.f) ? d.w : 0.f;
                } else {
                    const float4 a = make_float4(crelu01(x.x), crelu01(x.y), crelu01(x.z), crelu01(x.w));
                    g.x = d.x * ((a.x > 0.f && a.x < 1.f) ? 2.0f * a.x : 0.f);
                    g.y = d.y * ((a.y > 0.f && a.y < 1.f) ? 2.0f * a.y : 0.f);
                    g.z = d.z * ((a.z > 0.f && a.z < 1.f) ? 2.0f * a.z : 0.f);
                    g.w = d.w * ((a.w > 0.f && a.w < 1.f) ? 2.0f * a.w : 0.f);
                }
                store_dft(dft + ((size_t)pp * F + wcol) * ESZ, g);
                bacc0.x += g.x; bacc0.y += g.y; bacc0.z += g.z; bacc0.w += g.w;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    *reinterpret_cast<float4*>(bp + wcol) = bacc0;
    if (MODE == 1) *reinterpret_cast<float4*>(bp + half + wcol) = bacc1;
    if (HALF) {
        clamps = __reduce_add_sync(0xffffffffu, clamps);
        if ((threadIdx.x & 31) == 0 && clamps) atomicAdd(clamp_counter, (unsigned long long)clamps);
    }
}

// out[c] = sum over the perspectives (stm first) and the blocks' partial rows; 32 lanes share a column's rows and
// their partial sums are combined in lane order, a fixed order
__global__ void __launch_bounds__(256) k_bias_partials_reduce(const float* __restrict__ partials, int n_rows, int F,
                                                              float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // a warp per column
    if (c >= F) return;
    float sum = 0.f;
    const int total = 2 * n_rows;  // index i = p * n_rows + r
    for (int i = lane; i < total; i += 32) {
        const int p = i / n_rows, r = i - p * n_rows;
        sum += partials[((size_t)r * 2 + p) * F + c];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, d);
    if (lane == 0) out[c] = sum;
}

int launch_l1_dgrad_ftgrad(cudaStream_t s, int mode, const float* dl1, const int* order, const TileDesc* tiles,
                           const int* n_tiles, int max_tiles, const float* wb, const float* ws,
                           const void* pre_stm, const void* pre_nstm, const float* ft_bias, float scale,
                           int B, int F, int l1, int nb, void* dft_stm, void* dft_nstm, float* bias_partials,
                           float* ft_b_grad, int n_ctas, int half_act, float grad_scale, unsigned long long* clamp_counter) {
    (void)B;
    (void)max_tiles;
    const int work_cols = mode == 1 ? F / 2 : F;
    const int max_units = sort_max_units(max_tiles);
    int bias_rows = n_ctas;
    if ((l1 == 8 || l1 == 16 || l1 == 32) && n_ctas >= 2 * max_units) {
        int n_chunks = 1;
        while (work_cols / n_chunks > 1024 || (work_cols / n_chunks) % 128 != 0 && (work_cols / n_chunks) > 256) n_chunks *= 2;
        const int CW = work_cols / n_chunks;
        bias_rows = 2 * max_units;
        dim3 grid(bias_rows, 2, n_chunks), block(CW / 4);
        const size_t smem = (size_t)DG_STAGES * 4 * (mode == 1 ? 2 : 1) * (CW / 4) * (half_act ? 8 : 16);
#define DGRAD_REG(M, L, H)                                                                                               \
    do {                                                                                                                 \
        cudaFuncSetAttribute(k_l1_dgrad_ftgrad_stream<M, L, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
        k_l1_dgrad_ftgrad_stream<M, L, H><<<grid, block, smem, s>>>(dl1, order, tiles, tiles + max_tiles, n_tiles + 1, wb, ws, pre_stm, \
                                                                    pre_nstm, ft_bias, scale, F, nb, CW, dft_stm, dft_nstm, \
                                                                    bias_partials, grad_scale, clamp_counter);           \
    } while (0)
        if (half_act) {  // fp16 activations: LayerStack only
            if (mode != 1) return -1;
            if (l1 == 32) DGRAD_REG(1, 32, true); else if (l1 == 16) DGRAD_REG(1, 16, true); else DGRAD_REG(1, 8, true);
        }
        else if (l1 == 32) { if (mode == 1) DGRAD_REG(1, 32, false); else if (mode == 2) DGRAD_REG(2, 32, false); else DGRAD_REG(3, 32, false); }
        else if (l1 == 16) { if (mode == 1) DGRAD_REG(1, 16, false); else if (mode == 2) DGRAD_REG(2, 16, false); else DGRAD_REG(3, 16, false); }
        else { if (mode == 1) DGRAD_REG(1, 8, false); else if (mode == 2) DGRAD_REG(2, 8, false); else DGRAD_REG(3, 8, false); }
#undef DGRAD_REG
    } else {
        if (half_act) return -1;  // the fp16 activations need the streaming kernel (l1 of 8, 16 or 32)
        int n_chunks = 1;
        while ((size_t)(work_cols / n_chunks) * l1 * 4 > 64 * 1024 || work_cols / n_chunks > 1024) n_chunks *= 2;
        const int CW = work_cols / n_chunks;
        const size_t smem = (size_t)CW * l1 * sizeof(float);
        dim3 grid(n_ctas, 2, n_chunks), block(CW / 4);
#define DGRAD_LAUNCH(M)                                                                                                  \
    do {                                                                                                                 \
        cudaFuncSetAttribute(k_l1_dgrad_ftgrad<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);       \
        k_l1_dgrad_ftgrad<M><<<grid, block, smem, s>>>(dl1, order, tiles, n_tiles, wb, ws, static_cast<const float*>(pre_stm),  \
                                                         static_cast<const float*>(pre_nstm), ft_bias, scale, F, l1, nb, CW, \
                                                         static_cast<float*>(dft_stm), static_cast<float*>(dft_nstm), bias_partials); \
    } while (0)
        if (mode == 1) DGRAD_LAUNCH(1);
        else if (mode == 2) DGRAD_LAUNCH(2);
        else DGRAD_LAUNCH(3);
#undef DGRAD_LAUNCH
    }
    k_bias_partials_reduce<<<ceil_div(F, 8), 256, 0, s>>>(bias_partials, bias_rows, F, ft_b_grad);
    return 2;
}
