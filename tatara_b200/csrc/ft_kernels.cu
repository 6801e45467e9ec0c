// Sparse feature-transformer kernels: forward gather-sum (fused with the FT activation), inverse
// index, backward segmented reduce, factorizer reduce / fold.
//
// Layout: the FT table is row-major [rows, F] f32 (w[f*F + c], native_kernels.cu:162-200); every
// per-position tensor is row-major [B, F].  F is a multiple of 128, so rows are 512-byte aligned and
// every access below is a 128-bit vector.
#include "common.cuh"

#define SORT_KEYS_MAX 128  // key limit of the small-key sorts (sort_kernels.cu)

// ------------------------------------------------------------------------------------------------
// forward: one (position, perspective) item per group of F/8 threads.  Thread `lane` owns the float4
// at column 4*lane and its pair partner at column F/2 + 4*lane, so that the pairwise product of the
// LayerStack activation never leaves the thread.  Rows are added in slot order with plain f32 adds:
// the sums are bit-identical to sparse_ft_forward_cpu (sparse/sparse_ft_forward.rs:54-78).
// ------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(512) k_ft_forward(const float* __restrict__ table, const int* __restrict__ idx_stm,
                                                     const int* __restrict__ idx_nstm, const int* __restrict__ nnz,
                                                     const float* __restrict__ bias, float* __restrict__ pre_stm,
                                                     float* __restrict__ pre_nstm, float* __restrict__ combined,
                                                     const int* __restrict__ items, int n_items, int B, int F, int N, int A,
                                                     float scale, int ipc) {
    extern __shared__ int s_idx[];  // [ipc][A] indices, then [ipc] item ids
    int* s_item = s_idx + ipc * A;
    const int tpi = F >> 3;
    const int il = threadIdx.x / tpi;
    const int lane = threadIdx.x - il * tpi;
    const int slot0 = blockIdx.x * ipc;

    for (int i = threadIdx.x; i < ipc; i += blockDim.x) {
        const int sl = slot0 + i;
        s_item[i] = sl < n_items ? (items ? items[sl] : sl) : -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < ipc * A; i += blockDim.x) {
        const int li = i / A, a = i - li * A;
        const int it = s_item[li];
        int v = -1;
        if (it >= 0) {
            const int p = it >= B, b = it - p * B;
            if (a < nnz[b]) v = (p ? idx_nstm : idx_stm)[(size_t)b * A + a];
        }
        if ((unsigned)v >= (unsigned)N) v = -1;  // padding and out-of-range indices are skipped
        s_idx[i] = v;
    }
    __syncthreads();
    const int it = s_item[il];
    if (it < 0) return;
    const int persp = it >= B;
    const int item = it - persp * B;  // the position
    int n = nnz[item];
    n = n < 0 ? 0 : (n > A ? A : n);
    const int* my = s_idx + il * A;
    const float4* __restrict__ t4 = reinterpret_cast<const float4*>(table);
    const int row4 = F >> 2;
    const int c0 = lane, c1 = lane + tpi;

    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
    for (int a0 = 0; a0 < n; a0 += 8) {
        float4 va[8], vb[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int f = (a0 + u < n) ? my[a0 + u] : -1;
            if (f >= 0) {
                const float4* r = t4 + (size_t)f * row4;
                va[u] = __ldg(r + c0);
                vb[u] = __ldg(r + c1);
            } else {
                va[u] = make_float4(0.f, 0.f, 0.f, 0.f);  // x + 0.0 == x: a skipped slot leaves the sum unchanged
                vb[u] = va[u];
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            acc0.x += va[u].x; acc0.y += va[u].y; acc0.z += va[u].z; acc0.w += va[u].w;
            acc1.x += vb[u].x; acc1.y += vb[u].y; acc1.z += vb[u].z; acc1.w += vb[u].w;
        }
    }

    float4* pre = reinterpret_cast<float4*>(persp ? pre_nstm : pre_stm) + (size_t)item * row4;
    // outputs are written once and read by later kernels only: streaming stores leave L2 to the table slice
    if (MODE == 0) {
        __stcs(pre + c0, acc0);
        __stcs(pre + c1, acc1);
    } else if (MODE == 1) {
        // ft_post_perspective_fwd (layerstack/ft_post_perspective.rs:57-83): the raw sums are kept for the
        // backward pass, combined[b, persp*F/2 + r] = crelu(x_r + b_r) * crelu(x_{r+F/2} + b_{r+F/2}) * scale
        __stcs(pre + c0, acc0);
        __stcs(pre + c1, acc1);
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias) + c0);
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias) + c1);
        float4 o;
        o.x = crelu01(acc0.x + b0.x) * crelu01(acc1.x + b1.x) * scale;
        o.y = crelu01(acc0.y + b0.y) * crelu01(acc1.y + b1.y) * scale;
        o.z = crelu01(acc0.z + b0.z) * crelu01(acc1.z + b1.z) * scale;
        o.w = crelu01(acc0.w + b0.w) * crelu01(acc1.w + b1.w) * scale;
        __stcs(reinterpret_cast<float4*>(combined) + (size_t)item * row4 + persp * tpi + c0, o);
    } else {
        // simple_ft_post_fused_{crelu,screlu} (native_kernels.cu:1406-1450): the biased value replaces the
        // raw sum, combined[b, persp*F + c] = act(x)
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias) + c0);
        const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias) + c1);
        float4 x0 = make_float4(acc0.x + b0.x, acc0.y + b0.y, acc0.z + b0.z, acc0.w + b0.w);
        float4 x1 = make_float4(acc1.x + b1.x, acc1.y + b1.y, acc1.z + b1.z, acc1.w + b1.w);
        __stcs(pre + c0, x0);
        __stcs(pre + c1, x1);
        float4 a0 = make_float4(crelu01(x0.x), crelu01(x0.y), crelu01(x0.z), crelu01(x0.w));
        float4 a1 = make_float4(crelu01(x1.x), crelu01(x1.y), crelu01(x1.z), crelu01(x1.w));
        if (MODE == 3) {
            a0.x *= a0.x; a0.y *= a0.y; a0.z *= a0.z; a0.w *= a0.w;
            a1.x *= a1.x; a1.y *= a1.y; a1.z *= a1.z; a1.w *= a1.w;
        }
        float4* comb = reinterpret_cast<float4*>(combined) + (size_t)item * (2 * row4) + persp * row4;
        __stcs(comb + c0, a0);
        __stcs(comb + c1, a1);
    }
}

int launch_ft_forward(cudaStream_t s, int mode, const float* table, const int* idx_stm, const int* idx_nstm,
                      const int* nnz, const float* bias, float* pre_stm, float* pre_nstm, float* combined,
                      const int* items, int B, int F, int N, int A, float scale, int n_persp) {
    if (B <= 0) return 0;
    const int tpi = F / 8;
    int ipc = 256 / tpi;
    if (ipc < 1) ipc = 1;
    const int n_items = n_persp * B;
    dim3 grid(ceil_div(n_items, ipc)), block(ipc * tpi);
    size_t smem = (size_t)ipc * (A + 1) * sizeof(int);
#define FT_FWD_ARGS table, idx_stm, idx_nstm, nnz, bias, pre_stm, pre_nstm, combined, items, n_items, B, F, N, A, scale, ipc
    switch (mode) {
        case 0: k_ft_forward<0><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
        case 1: k_ft_forward<1><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
        case 2: k_ft_forward<2><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
        default: k_ft_forward<3><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
    }
#undef FT_FWD_ARGS
    return 1;
}

// ------------------------------------------------------------------------------------------------
// forward, slice-resident variant.  The generic kernel above gathers every row from L2; with the items sorted
// by king-bucket slice all of an item's rows lie in one slice of rows_per_slice rows, and a 32-column strip
// of that slice (rows_per_slice * 128 bytes, 208 KB for 1629 rows) fits in shared memory.  A block owns
// (run of <= 1024 items of one slice, column strip), loads the strip once and serves all of its items'
// row reads from shared memory; eight lanes work on one item, a lane on four adjacent columns (128-bit
// shared loads), rows are added in slot order as in the generic kernel, so the sums are bit-identical.
// A row outside the block's slice (arbitrary index lists) is read from the table in global memory instead.
// LayerStack strips hold columns [16s, 16s+16) and their pair partners [F/2 + 16s, F/2 + 16s + 16); the other
// modes 32 adjacent columns.
// ------------------------------------------------------------------------------------------------
#define SLICE_IPC 1024  // items per block
struct FwdWork {
    int slice, begin, end, pad;
};

__global__ void k_fwd_plan(const int* __restrict__ item_seg, int n_keys, FwdWork* __restrict__ work, int* __restrict__ n_work) {
    // n_keys = slices + 1 (the last key collects items without a usable first index)
    __shared__ int s_base[SORT_KEYS_MAX + 1];
    if (threadIdx.x == 0) {
        int run = 0;
        for (int k = 0; k < n_keys; ++k) {
            s_base[k] = run;
            run += (item_seg[k + 1] - item_seg[k] + SLICE_IPC - 1) / SLICE_IPC;
        }
        s_base[n_keys] = run;
        *n_work = run;
    }
    __syncthreads();
    for (int k = 0; k < n_keys; ++k) {
        const int b0 = item_seg[k], e0 = item_seg[k + 1];
        const int n = s_base[k + 1] - s_base[k];
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            FwdWork w;
            w.slice = k;
            w.begin = b0 + i * SLICE_IPC;
            w.end = min(e0, w.begin + SLICE_IPC);
            w.pad = 0;
            work[s_base[k] + i] = w;
        }
    }
}

template <int MODE, int NQ>
__global__ void __launch_bounds__(1024, 1) k_ft_forward_slice(const float* __restrict__ table, const int* __restrict__ idx_stm,
                                                               const int* __restrict__ idx_nstm, const int* __restrict__ nnz,
                                                               const float* __restrict__ bias, float* __restrict__ pre_stm,
                                                               float* __restrict__ pre_nstm, float* __restrict__ combined,
                                                               const int* __restrict__ items, const FwdWork* __restrict__ work,
                                                               const int* __restrict__ n_work, int B, int F, int N, int A, int rps,
                                                               int n_slices, float scale) {
    extern __shared__ __align__(16) float s_slice[];  // [rows][32]
    if ((int)blockIdx.x >= *n_work) return;
    const FwdWork wk = work[blockIdx.x];
    const int strip = blockIdx.y;
    const bool has_slice = wk.slice < n_slices;
    const int row0 = wk.slice * rps;
    const int rows = has_slice ? min(rps, N - row0) : 0;
    const int half = F >> 1;
    const int cA = MODE == 1 ? 16 * strip : 32 * strip;  // first column of the strip's first 16 (or all 32) columns
    const int cB = MODE == 1 ? half + 16 * strip : cA + 16;
    for (int e = threadIdx.x; e < rows * 8; e += blockDim.x) {
        const int r = e >> 3, q = e & 7;
        const int col = q < 4 ? cA + 4 * q : cB + 4 * (q - 4);
        *reinterpret_cast<float4*>(s_slice + r * 32 + 4 * q) =
            __ldg(reinterpret_cast<const float4*>(table + (size_t)(row0 + r) * F + col));
    }
    const int zero_row = rps * 32;  // float offset of one row of zeros behind the strip
    if (threadIdx.x < 32) s_slice[zero_row + threadIdx.x] = 0.f;
    __syncthreads();

    // eight lanes per item (a lane owns four adjacent columns: one 128-bit shared load per row), four items per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, j = lane & 7;
    const int mycol = j < 4 ? cA + 4 * j : cB + 4 * (j - 4);
    const float4 mybias = bias ? *reinterpret_cast<const float4*>(bias + mycol) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 pbias = mybias;  // the pair partner's bias (LayerStack)
    pbias.x = __shfl_xor_sync(0xffffffffu, mybias.x, 4); pbias.y = __shfl_xor_sync(0xffffffffu, mybias.y, 4);
    pbias.z = __shfl_xor_sync(0xffffffffu, mybias.z, 4); pbias.w = __shfl_xor_sync(0xffffffffu, mybias.w, 4);
    const float4* __restrict__ t4 = reinterpret_cast<const float4*>(table);
    // NQ index registers per lane: slots j, j + 8, ..., j + 8 (NQ - 1)
    const float* s_lane = s_slice + 4 * j;

    // software pipeline: item id two rounds ahead, its nnz and indices one round ahead
    auto load_item = [&](int slot) { return slot < wk.end ? __ldg(items + slot) : -1; };
    auto load_feats = [&](int it, int& n, int (&raw)[NQ]) {
        n = 0;
#pragma unroll
        for (int q = 0; q < NQ; ++q) raw[q] = -1;
        if (it >= 0) {
            const int p = it >= B, b = it - p * B;
            n = __ldg(nnz + b);
            const int* ip = (p ? idx_nstm : idx_stm) + (size_t)b * A;
#pragma unroll
            for (int q = 0; q < NQ; ++q)
                if (j + 8 * q < A) raw[q] = __ldg(ip + j + 8 * q);
        }
    };
    const int per_round = 4 * (blockDim.x >> 5);
    const int slot0 = wk.begin + 4 * warp + g;
    int it_c = load_item(slot0), it_n = load_item(slot0 + per_round);
    int n_c, raw_c[NQ];
    load_feats(it_c, n_c, raw_c);
    for (int base = wk.begin; base < wk.end; base += per_round) {
        const int it_n2 = load_item(base + 2 * per_round + 4 * warp + g);
        int n_n, raw_n[NQ];
        load_feats(it_n, n_n, raw_n);

        // ---- current item: indices -> shared-memory float offsets (>= 0), global fallback (<= -2) or skip (-1)
        const int n = n_c < 0 ? 0 : (n_c > A ? A : n_c);
        int code[NQ];
        bool outside = false;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            const int f = (j + 8 * q < n) ? raw_c[q] : -1;
            int c = zero_row;  // skipped slot: the all-zero row
            if ((unsigned)f < (unsigned)N) {
                const int r = f - row0;
                c = (unsigned)r < (unsigned)rows ? r * 32 : -(f + 2);
            }
            outside |= c < 0;
            code[q] = c;
        }
        int nmax = n;
        nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, 8));
        nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, 16));
        const bool slow = __any_sync(0xffffffffu, outside);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            if (8 * q >= nmax) break;
            if (!slow) {
                // every row of the round comes from the strip: branch-free; a skipped slot reads the all-zero row
                // kept behind the strip (x + 0.0 == x).  Two batches of four rows keep the register count low
                // enough for 32 warps per SM.
#pragma unroll
                for (int u0 = 0; u0 < 8; u0 += 4) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = __shfl_sync(0xffffffffu, code[q], (lane & 24) | (u0 + u));
                        v[u] = *reinterpret_cast<const float4*>(s_lane + c);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
                }
            } else {
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int c = __shfl_sync(0xffffffffu, code[q], (lane & 24) | u);
                    float4 v;
                    if (c >= 0) v = *reinterpret_cast<const float4*>(s_lane + c);
                    else v = __ldg(t4 + (((size_t)(-c - 2) * F + mycol) >> 2));
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
            }
        }

        // ---- epilogue
        const bool valid = it_c >= 0;
        const int persp = it_c >= B, b = valid ? it_c - persp * B : 0;
        float* pre = (persp ? pre_nstm : pre_stm) + (size_t)b * F;
        if (MODE == 0) {
            if (valid) __stcs(reinterpret_cast<float4*>(pre + mycol), acc);
        } else if (MODE == 1) {
            float4 pa;
            pa.x = __shfl_xor_sync(0xffffffffu, acc.x, 4); pa.y = __shfl_xor_sync(0xffffffffu, acc.y, 4);
            pa.z = __shfl_xor_sync(0xffffffffu, acc.z, 4); pa.w = __shfl_xor_sync(0xffffffffu, acc.w, 4);
            if (valid) {
                __stcs(reinterpret_cast<float4*>(pre + mycol), acc);
                if (j < 4) {
                    float4 o;
                    o.x = crelu01(acc.x + mybias.x) * crelu01(pa.x + pbias.x) * scale;
                    o.y = crelu01(acc.y + mybias.y) * crelu01(pa.y + pbias.y) * scale;
                    o.z = crelu01(acc.z + mybias.z) * crelu01(pa.z + pbias.z) * scale;
                    o.w = crelu01(acc.w + mybias.w) * crelu01(pa.w + pbias.w) * scale;
                    __stcs(reinterpret_cast<float4*>(combined + (size_t)b * F + persp * half + cA + 4 * j), o);
                }
            }
        } else if (valid) {
            const float4 x = make_float4(acc.x + mybias.x, acc.y + mybias.y, acc.z + mybias.z, acc.w + mybias.w);
            __stcs(reinterpret_cast<float4*>(pre + mycol), x);
            float4 a = make_float4(crelu01(x.x), crelu01(x.y), crelu01(x.z), crelu01(x.w));
            if (MODE == 3) { a.x *= a.x; a.y *= a.y; a.z *= a.z; a.w *= a.w; }
            __stcs(reinterpret_cast<float4*>(combined + (size_t)b * 2 * F + persp * F + mycol), a);
        }
        it_c = it_n; it_n = it_n2; n_c = n_n;
#pragma unroll
        for (int q = 0; q < NQ; ++q) raw_c[q] = raw_n[q];
    }
}

// work: [ceil(n_items / 1024) + keys + 1] FwdWork records followed by one int (their count)
size_t ft_forward_slice_work_ints(int n_items, int n_keys) { return 4 * ((size_t)n_items / SLICE_IPC + n_keys + 2) + 4; }

bool ft_forward_slice_supported(int F, int N, int A, int rps) {
    int n_slices = ceil_div(N, rps);
    return F % 32 == 0 && A <= 64 && ((size_t)rps + 1) * 128 <= 226 * 1024 && n_slices + 1 <= SORT_KEYS_MAX;
}

int launch_ft_forward_slice(cudaStream_t s, int mode, const float* table, const int* idx_stm, const int* idx_nstm,
                            const int* nnz, const float* bias, float* pre_stm, float* pre_nstm, float* combined,
                            const int* items, const int* item_seg, int* work, int B, int F, int N, int A, int rps,
                            float scale, int n_persp) {
    if (B <= 0) return 0;
    const int n_items = n_persp * B;
    const int n_slices = ceil_div(N, rps), n_keys = n_slices + 1;
    const int max_work = n_items / SLICE_IPC + n_keys + 2;
    FwdWork* wk = reinterpret_cast<FwdWork*>(work);
    int* n_work = work + 4 * (size_t)max_work;
    k_fwd_plan<<<1, 128, 0, s>>>(item_seg, n_keys, wk, n_work);
    const size_t smem = ((size_t)rps + 1) * 32 * sizeof(float);  // the strip and one row of zeros
    dim3 grid(max_work, F / 32);
#define FT_SLICE_ARGS table, idx_stm, idx_nstm, nnz, bias, pre_stm, pre_nstm, combined, items, wk, n_work, B, F, N, A, rps, n_slices, scale
#define FT_SLICE_LAUNCH(M, Q)                                                                                      \
    do {                                                                                                           \
        cudaFuncSetAttribute(k_ft_forward_slice<M, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        k_ft_forward_slice<M, Q><<<grid, 1024, smem, s>>>(FT_SLICE_ARGS);                                          \
    } while (0)
    const bool q5 = A <= 40;
    switch (mode) {
        case 0: if (q5) FT_SLICE_LAUNCH(0, 5); else FT_SLICE_LAUNCH(0, 8); break;
        case 1: if (q5) FT_SLICE_LAUNCH(1, 5); else FT_SLICE_LAUNCH(1, 8); break;
        case 2: if (q5) FT_SLICE_LAUNCH(2, 5); else FT_SLICE_LAUNCH(2, 8); break;
        default: if (q5) FT_SLICE_LAUNCH(3, 5); else FT_SLICE_LAUNCH(3, 8); break;
    }
#undef FT_SLICE_LAUNCH
#undef FT_SLICE_ARGS
    return 2;
}

// ------------------------------------------------------------------------------------------------
// inverse index: for every feature the list of positions that hold it (the counting sort of
// native_kernels.cu:1630-1765: histogram, exclusive scan, ranked scatter).
// ------------------------------------------------------------------------------------------------
__global__ void k_feat_count(const int* __restrict__ idx_stm, const int* __restrict__ idx_nstm,
                             const int* __restrict__ nnz, int B, int A, int N, int n_persp, int* __restrict__ counts) {
    const long long total = (long long)n_persp * B * A;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(i / ((long long)B * A));
        const long long r = i - (long long)p * B * A;
        const int b = (int)(r / A), a = (int)(r - (long long)b * A);
        if (a >= nnz[b]) continue;
        const int f = (p ? idx_nstm : idx_stm)[r];
        if ((unsigned)f < (unsigned)N) atomicAdd(counts + (size_t)p * N + f, 1);
    }
}

// offsets[p][0..N] = exclusive prefix sum of counts[p][0..N), in two launches: block-local scans of 2048
// cells with their sums, then every block adds the sums of the blocks before it.
#define SCAN_CELLS 2048
__global__ void __launch_bounds__(1024) k_feat_scan_local(const int* __restrict__ counts, int N, int* __restrict__ offsets,
                                                           int* __restrict__ block_sums) {
    __shared__ int warp_tot[32];
    const int p = blockIdx.y;
    const int* c = counts + (size_t)p * N;
    int* o = offsets + (size_t)p * (N + 1);
    const int i0 = blockIdx.x * SCAN_CELLS + 2 * threadIdx.x;
    const int a = i0 < N ? c[i0] : 0, b = i0 + 1 < N ? c[i0 + 1] : 0;
    const int sum = a + b;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) warp_tot[w] = incl;
    __syncthreads();
    if (w == 0) {
        const int t = warp_tot[lane];
        int ti = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, ti, d);
            if (lane >= d) ti += u;
        }
        warp_tot[lane] = ti - t;
        if (lane == 31) block_sums[p * gridDim.x + blockIdx.x] = ti;
    }
    __syncthreads();
    const int excl = warp_tot[w] + incl - sum;
    if (i0 < N) o[i0] = excl;
    if (i0 + 1 < N) o[i0 + 1] = excl + a;
}

__global__ void __launch_bounds__(1024) k_feat_scan_add(int N, int* __restrict__ offsets, int* __restrict__ cursor,
                                                         const int* __restrict__ block_sums) {
    __shared__ int s_off;
    const int p = blockIdx.y;
    int* o = offsets + (size_t)p * (N + 1);
    int* cur = cursor + (size_t)p * N;
    if (threadIdx.x < 32) {
        int t = 0;
        for (int j = threadIdx.x; j < (int)blockIdx.x; j += 32) t += block_sums[p * gridDim.x + j];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) t += __shfl_down_sync(0xffffffffu, t, d);
        if (threadIdx.x == 0) s_off = t;
    }
    __syncthreads();
    const int off = s_off;
    const int i0 = blockIdx.x * SCAN_CELLS + 2 * threadIdx.x;
    if (i0 < N) { const int v = o[i0] + off; o[i0] = v; cur[i0] = v; }
    if (i0 + 1 < N) { const int v = o[i0 + 1] + off; o[i0 + 1] = v; cur[i0 + 1] = v; }
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) o[N] = off + block_sums[p * gridDim.x + blockIdx.x];
}

__global__ void k_feat_fill(const int* __restrict__ idx_stm, const int* __restrict__ idx_nstm,
                            const int* __restrict__ nnz, int B, int A, int N, int n_persp, int* __restrict__ cursor,
                            int* __restrict__ lists) {
    const long long total = (long long)n_persp * B * A;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int p = (int)(i / ((long long)B * A));
        const long long r = i - (long long)p * B * A;
        const int b = (int)(r / A), a = (int)(r - (long long)b * A);
        if (a >= nnz[b]) continue;
        const int f = (p ? idx_nstm : idx_stm)[r];
        if ((unsigned)f < (unsigned)N) {
            const int pos = atomicAdd(cursor + (size_t)p * N + f, 1);
            lists[(size_t)p * B * A + pos] = b;
        }
    }
}

// The ranked scatter above leaves every list in arrival order.  The two kernels below sort each list
// ascending, so that the backward sums always run in position order (deterministic results).
// Short lists (<= 64 entries): one warp ranks its entries against each other through shuffles.
// Long lists: queued, then one block per list marks the positions in a shared-memory bitmap and reads
// the set bits back in order; a list that names a position twice (only possible when the caller's
// index row repeats a feature) falls back to ranking by counting.
__global__ void __launch_bounds__(256) k_lists_sort_short(const int* __restrict__ offsets, int N, int n_persp, int B, int A,
                                                           int* __restrict__ lists, int* __restrict__ long_queue,
                                                           int* __restrict__ long_count) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_persp * N) return;
    const int p = warp / N, f = warp - p * N;
    const int beg = offsets[(size_t)p * (N + 1) + f], end = offsets[(size_t)p * (N + 1) + f + 1];
    const int len = end - beg;
    if (len < 2) return;
    if (len > 64) {
        if (lane == 0) long_queue[atomicAdd(long_count, 1)] = warp;
        return;
    }
    int* L = lists + (size_t)p * B * A + beg;
    const int v0 = lane < len ? L[lane] : 0x7fffffff;
    const int v1 = lane + 32 < len ? L[lane + 32] : 0x7fffffff;
    int r0 = 0, r1 = 0;
    for (int j = 0; j < len; ++j) {
        const int u = __shfl_sync(0xffffffffu, j < 32 ? v0 : v1, j & 31);
        r0 += (u < v0) || (u == v0 && j < lane);
        r1 += (u < v1) || (u == v1 && j < lane + 32);
    }
    __syncwarp();
    if (lane < len) L[r0] = v0;
    if (lane + 32 < len) L[r1] = v1;
}

__global__ void __launch_bounds__(256) k_lists_sort_long(const int* __restrict__ offsets, int N, int B, int A,
                                                          int* __restrict__ lists, int* __restrict__ scratch,
                                                          const int* __restrict__ long_queue,
                                                          const int* __restrict__ long_count, int bitmap_words) {
    extern __shared__ unsigned s_bits[];  // [bitmap_words]; 0 words: always use the counting fallback
    __shared__ int s_warp[8];
    __shared__ int s_total;
    const int n_long = *long_count;
    for (int q = blockIdx.x; q < n_long; q += gridDim.x) {
        const int id = long_queue[q];
        const int p = id / N, f = id - p * N;
        const int beg = offsets[(size_t)p * (N + 1) + f], end = offsets[(size_t)p * (N + 1) + f + 1];
        const int len = end - beg;
        int* L = lists + (size_t)p * B * A + beg;
        bool done = false;
        if (bitmap_words > 0) {
            for (int i = threadIdx.x; i < bitmap_words; i += blockDim.x) s_bits[i] = 0u;
            __syncthreads();
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                const int b = L[i];
                atomicOr(&s_bits[b >> 5], 1u << (b & 31));
            }
            __syncthreads();
            const int per = (bitmap_words + blockDim.x - 1) / blockDim.x;
            const int w0 = threadIdx.x * per, w1 = min(w0 + per, bitmap_words);
            int cnt = 0;
            for (int w = w0; w < w1; ++w) cnt += __popc(s_bits[w]);
            // block exclusive scan of cnt
            const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
            int incl = cnt;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += t;
            }
            if (lane == 31) s_warp[wid] = incl;
            __syncthreads();
            if (threadIdx.x == 0) {
                int run = 0;
                for (int i = 0; i < 8; ++i) { int t = s_warp[i]; s_warp[i] = run; run += t; }
                s_total = run;
            }
            __syncthreads();
            if (s_total == len) {
                int pos = s_warp[wid] + incl - cnt;
                for (int w = w0; w < w1; ++w) {
                    unsigned bits = s_bits[w];
                    while (bits) {
                        const int bit = __ffs(bits) - 1;
                        bits &= bits - 1;
                        L[pos++] = (w << 5) + bit;
                    }
                }
                done = true;
            }
            __syncthreads();
        }
        if (!done) {
            int* S = scratch + (size_t)p * B * A + beg;
            for (int i = threadIdx.x; i < len; i += blockDim.x) S[i] = L[i];
            __syncthreads();
            for (int i = threadIdx.x; i < len; i += blockDim.x) {
                const int v = S[i];
                int r = 0;
                for (int j = 0; j < len; ++j) {
                    const int u = S[j];
                    r += (u < v) || (u == v && j < i);
                }
                L[r] = v;
            }
            __syncthreads();
        }
    }
}

int launch_inverse_index(cudaStream_t s, const int* idx_stm, const int* idx_nstm, const int* nnz, int B, int A,
                         int N, int n_persp, int* counts, int* offsets, int* cursor, int* lists) {
    if (B <= 0) return 0;
    // counts holds [2][N] histogram cells followed by one counter and a queue of [2*N] long-list ids
    int* long_count = counts + (size_t)2 * N;
    int* long_queue = long_count + 1;
    cudaMemsetAsync(counts, 0, sizeof(int) * ((size_t)2 * N + 1), s);
    const long long total = (long long)n_persp * B * A;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    k_feat_count<<<blocks, 256, 0, s>>>(idx_stm, idx_nstm, nnz, B, A, N, n_persp, counts);
    {   // block sums live behind the long-list queue (which holds at most 2N ids)
        int* block_sums = long_queue + (size_t)2 * N;
        const dim3 sg(ceil_div(N, SCAN_CELLS), n_persp);
        k_feat_scan_local<<<sg, 1024, 0, s>>>(counts, N, offsets, block_sums);
        k_feat_scan_add<<<sg, 1024, 0, s>>>(N, offsets, cursor, block_sums);
    }
    k_feat_fill<<<blocks, 256, 0, s>>>(idx_stm, idx_nstm, nnz, B, A, N, n_persp, cursor, lists);
    int* scratch = lists + (size_t)2 * B * A;  // the list buffer carries a second copy's worth of room
    const long long warps = (long long)n_persp * N;
    k_lists_sort_short<<<(int)((warps * 32 + 255) / 256), 256, 0, s>>>(offsets, N, n_persp, B, A, lists, long_queue, long_count);
    int words = (B + 31) / 32;
    if ((size_t)words * 4 > 160 * 1024) words = 0;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(k_lists_sort_long, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        attr_set = true;
    }
    k_lists_sort_long<<<148 * 4, 256, (size_t)words * 4, s>>>(offsets, N, B, A, lists, scratch, long_queue, long_count, words);
    return 6;
}

// ------------------------------------------------------------------------------------------------
// backward: one block per feature row, one thread per float4 column.  The row of the gradient is
// written exactly once per step (stm list first, then nstm list, each in ascending position order —
// the accumulation order of sparse_ft_backward_cpu called for stm then nstm).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512) k_ft_backward(const float* __restrict__ dft_stm, const float* __restrict__ dft_nstm,
                                                       const int* __restrict__ offsets, const int* __restrict__ lists,
                                                       int B, int A, int N, int F, int n_persp, float* __restrict__ grad) {
    const int f = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int row4 = F >> 2;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < n_persp; ++p) {
        const int beg = offsets[(size_t)p * (N + 1) + f], end = offsets[(size_t)p * (N + 1) + f + 1];
        const int* __restrict__ L = lists + (size_t)p * B * A;
        const float4* __restrict__ d = reinterpret_cast<const float4*>(p ? dft_nstm : dft_stm);
        for (int j = beg; j < end; j += 8) {
            // unconditional loads (a slot past the end re-reads the last row and is dropped below), so that all
            // eight row loads are in flight together
            int bi[8];
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) bi[u] = __ldg(L + min(j + u, end - 1));
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldg(d + (size_t)bi[u] * row4 + c);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (j + u < end) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
            }
        }
    }
    reinterpret_cast<float4*>(grad)[(size_t)f * row4 + c] = acc;
}

int launch_ft_backward(cudaStream_t s, const float* dft_stm, const float* dft_nstm, const int* offsets,
                       const int* lists, int B, int A, int N, int F, int n_persp, float* grad) {
    const int ny = ceil_div(F / 4, 512), bx = F / 4 / ny;  // at most 512 threads per block: room for 64 registers each
    k_ft_backward<<<dim3(N, ny), bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, grad);
    return 1;
}

// ------------------------------------------------------------------------------------------------
// backward with list splitting.  A feature that is active in very many positions (the king square of a
// king bucket, a pawn in hand) makes one block walk a list of thousands of rows; with real, skewed data such
// lists reach tens of thousands of entries and would set the kernel's run time on their own.  Features whose
// lists (stm + nstm) exceed BWD_PART entries are cut into parts of BWD_PART entries; every part is summed
// by its own block into a scratch row, and a last kernel adds the parts of a feature in order.  Which
// block gets which part depends on timing, the sums do not.
// ------------------------------------------------------------------------------------------------
#define BWD_PART 4096

__global__ void k_bwd_plan(const int* __restrict__ offsets, int N, int n_persp, int* __restrict__ counters,
                           int2* __restrict__ work, int* __restrict__ longf) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= N) return;
    int len = 0;
    for (int p = 0; p < n_persp; ++p) len += offsets[(size_t)p * (N + 1) + f + 1] - offsets[(size_t)p * (N + 1) + f];
    if (len <= BWD_PART) return;
    const int parts = (len + BWD_PART - 1) / BWD_PART;
    const int base = atomicAdd(&counters[0], parts);
    const int q = atomicAdd(&counters[1], 1);
    longf[3 * q + 0] = f;
    longf[3 * q + 1] = base;
    longf[3 * q + 2] = parts;
    for (int i = 0; i < parts; ++i) work[base + i] = make_int2(f, i);
}

static __device__ __forceinline__ float4 sum_rows(const float4* __restrict__ d, const int* __restrict__ L, int beg, int end,
                                                  int row4, int c, float4 acc) {
    for (int j = beg; j < end; j += 8) {
        int bi[8];
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) bi[u] = __ldg(L + min(j + u, end - 1));
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(d + (size_t)bi[u] * row4 + c);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (j + u < end) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
        }
    }
    return acc;
}

__global__ void __launch_bounds__(512) k_ft_backward_short(const float* __restrict__ dft_stm, const float* __restrict__ dft_nstm,
                                                             const int* __restrict__ offsets, const int* __restrict__ lists,
                                                             int B, int A, int N, int F, int n_persp, float* __restrict__ grad) {
    const int f = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int row4 = F >> 2;
    int len = offsets[f + 1] - offsets[f];
    if (n_persp > 1) len += offsets[(size_t)(N + 1) + f + 1] - offsets[(size_t)(N + 1) + f];
    if (len > BWD_PART) return;  // summed in parts by k_ft_backward_long
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < n_persp; ++p) {
        const int beg = offsets[(size_t)p * (N + 1) + f], end = offsets[(size_t)p * (N + 1) + f + 1];
        const int* __restrict__ L = lists + (size_t)p * B * A;
        const float4* __restrict__ d = reinterpret_cast<const float4*>(p ? dft_nstm : dft_stm);
        for (int j = beg; j < end; j += 8) {
            // unconditional loads (a slot past the end re-reads the last row and is dropped below), so that all
            // eight row loads are in flight together
            int bi[8];
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) bi[u] = __ldg(L + min(j + u, end - 1));
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldg(d + (size_t)bi[u] * row4 + c);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (j + u < end) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
            }
        }
    }
    reinterpret_cast<float4*>(grad)[(size_t)f * row4 + c] = acc;
}

__global__ void __launch_bounds__(512) k_ft_backward_long(const float* __restrict__ dft_stm, const float* __restrict__ dft_nstm,
                                                            const int* __restrict__ offsets, const int* __restrict__ lists,
                                                            int B, int A, int N, int F, int n_persp,
                                                            const int* __restrict__ counters, const int2* __restrict__ work,
                                                            float* __restrict__ partial) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int row4 = F >> 2;
    const int n_work = counters[0];
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
        const int2 wk = work[w];
        const int f = wk.x;
        int lo = wk.y * BWD_PART, hi = lo + BWD_PART;  // range in the concatenated (stm, nstm) list
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < n_persp; ++p) {
            const int beg = offsets[(size_t)p * (N + 1) + f], len = offsets[(size_t)p * (N + 1) + f + 1] - beg;
            const int a = max(lo, 0), b = min(hi, len);
            if (a < b)
                acc = sum_rows(reinterpret_cast<const float4*>(p ? dft_nstm : dft_stm), lists + (size_t)p * B * A, beg + a, beg + b,
                               row4, c, acc);
            lo -= len;
            hi -= len;
        }
        reinterpret_cast<float4*>(partial)[(size_t)w * row4 + c] = acc;
    }
}

__global__ void __launch_bounds__(512) k_ft_backward_long_final(const int* __restrict__ counters, const int* __restrict__ longf,
                                                                  const float* __restrict__ partial, int F,
                                                                  float* __restrict__ grad) {
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int row4 = F >> 2;
    const int n_long = counters[1];
    const float4* p4 = reinterpret_cast<const float4*>(partial);
    for (int q = blockIdx.x; q < n_long; q += gridDim.x) {
        const int f = longf[3 * q], base = longf[3 * q + 1], parts = longf[3 * q + 2];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < parts; ++i) {
            const float4 v = p4[(size_t)(base + i) * row4 + c];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(grad)[(size_t)f * row4 + c] = acc;
    }
}

int ft_backward_max_work(int B, int A, int n_persp) { return 2 * (int)(((long long)n_persp * B * A) / BWD_PART) + 2; }

// plan: [2] counters, then [2 * max_work] work items, then [3 * N] long-feature records; partial: [max_work][F]
int launch_ft_backward_split(cudaStream_t s, const float* dft_stm, const float* dft_nstm, const int* offsets,
                             const int* lists, int B, int A, int N, int F, int n_persp, int* plan, float* partial,
                             float* grad) {
    const int max_work = ft_backward_max_work(B, A, n_persp);
    int* counters = plan;
    int2* work = reinterpret_cast<int2*>(plan + 2);
    int* longf = plan + 2 + 2 * max_work;
    cudaMemsetAsync(counters, 0, 2 * sizeof(int), s);
    k_bwd_plan<<<ceil_div(N, 256), 256, 0, s>>>(offsets, N, n_persp, counters, work, longf);
    const int ny = ceil_div(F / 4, 512), bx = F / 4 / ny;  // at most 512 threads per block: room for 64 registers each
    k_ft_backward_short<<<dim3(N, ny), bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, grad);
    k_ft_backward_long<<<dim3(148 * 4, ny), bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, counters, work, partial);
    k_ft_backward_long_final<<<dim3(148 * 2, ny), bx, 0, s>>>(counters, longf, partial, F, grad);
    return 4;
}

// ft_reduce_virtual_grad (sparse/ft_factorize.rs:109-121): grad[N + v] = sum over king buckets of grad[kb*pi + v]
__global__ void k_ft_reduce_virtual(float* __restrict__ grad, int N, int pi, int F) {
    const int row4 = F >> 2;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)pi * row4) return;
    const int v = (int)(i / row4), c = (int)(i - (long long)v * row4);
    const float4* g4 = reinterpret_cast<const float4*>(grad);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int f = v; f < N; f += pi) {
        const float4 x = g4[(size_t)f * row4 + c];
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    reinterpret_cast<float4*>(grad)[(size_t)(N + v) * row4 + c] = acc;
}

int launch_ft_reduce_virtual(cudaStream_t s, float* grad, int N, int pi, int F) {
    const long long n = (long long)pi * (F / 4);
    k_ft_reduce_virtual<<<(int)((n + 255) / 256), 256, 0, s>>>(grad, N, pi, F);
    return 1;
}

// ft_fold_virtual (sparse/ft_factorize.rs:78-99): comb[f] = w[f] + w[N + f % pi]
__global__ void k_ft_fold(const float* __restrict__ w, float* __restrict__ comb, int N, int pi, int F) {
    const int row4 = F >> 2;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)N * row4) return;
    const int f = (int)(i / row4), c = (int)(i - (long long)f * row4);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const float4 a = w4[i];
    const float4 b = w4[(size_t)(N + f % pi) * row4 + c];
    reinterpret_cast<float4*>(comb)[i] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
}

int launch_ft_fold(cudaStream_t s, const float* w, float* comb, int N, int pi, int F) {
    const long long n = (long long)N * (F / 4);
    k_ft_fold<<<(int)((n + 255) / 256), 256, 0, s>>>(w, comb, N, pi, F);
    return 1;
}
