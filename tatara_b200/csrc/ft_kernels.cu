// Sparse feature-transformer kernels: forward gather-sum (fused with the FT activation), inverse
// index, backward segmented reduce, factorizer reduce / fold.
//
// Layout: the FT table is row-major [rows, F] f32 (w[f*F + c], native_kernels.cu:162-200); every
// per-position tensor is row-major [B, F].  F is a multiple of 128, so rows are 512-byte aligned and
// every access below is a 128-bit vector.
#include "common.cuh"
#include "ft_slice.cuh"
#include <stdlib.h>

#define SORT_KEYS_MAX 128  // key limit of the small-key sorts (sort_kernels.cu)

// ------------------------------------------------------------------------------------------------
// forward: one (position, perspective) item per group of F/8 threads.  Thread `lane` owns the float4
// at column 4*lane and its pair partner at column F/2 + 4*lane, so that the pairwise product of the
// LayerStack activation never leaves the thread.  Rows are added in slot order with plain f32 adds:
// the sums are bit-identical to sparse_ft_forward_cpu (sparse/sparse_ft_forward.rs:54-78).
// ------------------------------------------------------------------------------------------------
// four consecutive table / activation values as fp32, whatever their storage type
template <bool H>
static __device__ __forceinline__ float4 ld4(const void* base, size_t elem) {
    if (H) {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(base) + elem));
        const float2 a = unpack_h2(u.x), b = unpack_h2(u.y);
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem));
}
template <bool H>
static __device__ __forceinline__ void st4_cs(void* base, size_t elem, float4 v) {
    if (H) __stcs(reinterpret_cast<uint2*>(static_cast<__half*>(base) + elem), make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w)));
    else __stcs(reinterpret_cast<float4*>(static_cast<float*>(base) + elem), v);
}
static __device__ __forceinline__ float4 round_h4(float4 v) {
    const float2 a = unpack_h2(pack_h2(v.x, v.y)), b = unpack_h2(pack_h2(v.z, v.w));
    return make_float4(a.x, a.y, b.x, b.y);
}

// TH: fp16 table rows (summed in fp32); OH: fp16 pre-activations, the activation computed from the rounded values
template <int MODE, bool TH, bool OH>
__global__ void __launch_bounds__(512) k_ft_forward(const void* __restrict__ table, const int* __restrict__ idx_stm,
                                                     const int* __restrict__ idx_nstm, const int* __restrict__ nnz,
                                                     const float* __restrict__ bias, void* __restrict__ pre_stm,
                                                     void* __restrict__ pre_nstm, float* __restrict__ combined,
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
    const int row4 = F >> 2;
    const int c0 = lane, c1 = lane + tpi;

    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
    for (int a0 = 0; a0 < n; a0 += 8) {
        float4 va[8], vb[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int f = (a0 + u < n) ? my[a0 + u] : -1;
            if (f >= 0) {
                va[u] = ld4<TH>(table, (size_t)f * F + 4 * c0);
                vb[u] = ld4<TH>(table, (size_t)f * F + 4 * c1);
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

    void* pre = persp ? pre_nstm : pre_stm;
    const size_t e0 = (size_t)item * F + 4 * c0, e1 = (size_t)item * F + 4 * c1;
    if (OH) { acc0 = round_h4(acc0); acc1 = round_h4(acc1); }
    // outputs are written once and read by later kernels only: streaming stores leave L2 to the table slice
    if (MODE == 0) {
        st4_cs<OH>(pre, e0, acc0);
        st4_cs<OH>(pre, e1, acc1);
    } else if (MODE == 1) {
        // ft_post_perspective_fwd (layerstack/ft_post_perspective.rs:57-83): the raw sums are kept for the
        // backward pass, combined[b, persp*F/2 + r] = crelu(x_r + b_r) * crelu(x_{r+F/2} + b_{r+F/2}) * scale
        st4_cs<OH>(pre, e0, acc0);
        st4_cs<OH>(pre, e1, acc1);
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
        st4_cs<OH>(pre, e0, x0);
        st4_cs<OH>(pre, e1, x1);
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

int launch_ft_forward(cudaStream_t s, int mode, const void* table, const int* idx_stm, const int* idx_nstm,
                      const int* nnz, const float* bias, void* pre_stm, void* pre_nstm, float* combined,
                      const int* items, int B, int F, int N, int A, float scale, int n_persp, int table_half, int out_half) {
    if (B <= 0) return 0;
    const int tpi = F / 8;
    int ipc = 256 / tpi;
    if (ipc < 1) ipc = 1;
    const int n_items = n_persp * B;
    dim3 grid(ceil_div(n_items, ipc)), block(ipc * tpi);
    size_t smem = (size_t)ipc * (A + 1) * sizeof(int);
#define FT_FWD_ARGS table, idx_stm, idx_nstm, nnz, bias, pre_stm, pre_nstm, combined, items, n_items, B, F, N, A, scale, ipc
    if (table_half) {
        if (mode == 0 && !out_half) k_ft_forward<0, true, false><<<grid, block, smem, s>>>(FT_FWD_ARGS);
        else if (mode == 1 && !out_half) k_ft_forward<1, true, false><<<grid, block, smem, s>>>(FT_FWD_ARGS);
        else if (mode == 1) k_ft_forward<1, true, true><<<grid, block, smem, s>>>(FT_FWD_ARGS);
        else return -1;
        return 1;
    }
    if (out_half) return -1;
    switch (mode) {
        case 0: k_ft_forward<0, false, false><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
        case 1: k_ft_forward<1, false, false><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
        case 2: k_ft_forward<2, false, false><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
        default: k_ft_forward<3, false, false><<<grid, block, smem, s>>>(FT_FWD_ARGS); break;
    }
#undef FT_FWD_ARGS
    return 1;
}

// ------------------------------------------------------------------------------------------------
// forward, slice-resident variant.  The generic kernel above gathers every row from L2; with the items sorted
// by king-bucket slice all of an item's rows lie in one slice of rows_per_slice rows, and a 32-column strip
// of that slice (rows_per_slice * 128 bytes, 208 KB for 1629 rows) fits in shared memory.  A block owns
// (run of <= SLICE_IPC items of one slice, column strip), loads the strip once and serves all of its items'
// row reads from shared memory; eight lanes work on one item, a lane on four adjacent columns (128-bit
// shared loads), rows are added in slot order as in the generic kernel, so the sums are bit-identical.
// A row outside the block's slice (arbitrary index lists) is read from the table in global memory instead.
// LayerStack strips hold columns [16s, 16s+16) and their pair partners [F/2 + 16s, F/2 + 16s + 16); the other
// modes 32 adjacent columns.
// ------------------------------------------------------------------------------------------------
__global__ void k_fwd_plan(const int* __restrict__ item_seg, int n_keys, int ipc, FwdWork* __restrict__ work, int* __restrict__ n_work) {
    // n_keys = slices + 1 (the last key collects items without a usable first index)
    __shared__ int s_base[SORT_KEYS_MAX + 1], s_seg[SORT_KEYS_MAX + 2];
    for (int k = threadIdx.x; k <= n_keys; k += blockDim.x) s_seg[k] = item_seg[k];  // one round trip, not n_keys
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int k = 0; k < n_keys; ++k) {
            s_base[k] = run;
            run += (s_seg[k + 1] - s_seg[k] + ipc - 1) / ipc;
        }
        s_base[n_keys] = run;
        n_work[0] = run;
        n_work[1] = 0;  // "some item has a row outside its slice", raised by k_fwd_codes
    }
    __syncthreads();
    for (int k = 0; k < n_keys; ++k) {
        const int b0 = s_seg[k], e0 = s_seg[k + 1];
        const int n = s_base[k + 1] - s_base[k];
        // equal runs, a multiple of the 128 items a block handles per round (<= ipc, itself such a multiple)
        const int size = n > 0 ? ((e0 - b0 + n - 1) / n + 127) & ~127 : 0;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            FwdWork w;
            w.slice = k;
            w.begin = min(e0, b0 + i * size);
            w.end = min(e0, w.begin + size);
            w.pad = 0;
            work[s_base[k] + i] = w;
        }
    }
}

// Row codes of the slice-resident forward, one thread per slot of the sorted item list: for every feature slot the
// row number inside the item's slice (16 bits), SLICE_ZERO_ROW's stand-in rps for a slot without a feature (the strip
// keeps a row of zeros there), SLICE_OUTSIDE for a table row outside the slice (the kernel then reads the index list).
// info[slot] = item | SLICE_SLOW_BIT when the item has an outside row.  Codes of consecutive slots are contiguous
// (A_pad 16-bit codes each, A_pad a multiple of 8), so a warp copies its round of four items in 16-byte pieces.
__global__ void __launch_bounds__(256) k_fwd_codes(const int* __restrict__ idx_stm, const int* __restrict__ idx_nstm,
                                                   const int* __restrict__ nnz, const int* __restrict__ items,
                                                   const int* __restrict__ item_seg, int n_keys, int n_items, int B, int N,
                                                   int A, int A_pad, int rps, uint4* __restrict__ codes,
                                                   int* __restrict__ info, int* __restrict__ outside_flag) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n_items) return;
    int lo = 0, hi = n_keys - 1;  // the key whose segment holds slot s
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(item_seg + mid) <= s) lo = mid; else hi = mid - 1;
    }
    const int row0 = lo * rps;
    const int rows = max(0, min(rps, N - row0));
    const int it = __ldg(items + s);
    const int p = it >= B, b = it - p * B;
    int n = __ldg(nnz + b);
    n = n < 0 ? 0 : (n > A ? A : n);
    const int* ip = (p ? idx_nstm : idx_stm) + (size_t)b * A;
    bool outside = false;
    for (int q0 = 0; q0 < A_pad; q0 += 8) {
        unsigned c[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int q = q0 + u;
            unsigned code = (unsigned)rps;
            if (q < n) {
                const int f = __ldg(ip + q);
                if ((unsigned)f < (unsigned)N) {
                    const int r = f - row0;
                    if ((unsigned)r < (unsigned)rows) code = (unsigned)r;
                    else { code = SLICE_OUTSIDE; outside = true; }
                }
            }
            c[u] = code;
        }
        codes[((size_t)s * A_pad + q0) >> 3] = make_uint4(c[0] | (c[1] << 16), c[2] | (c[3] << 16), c[4] | (c[5] << 16), c[6] | (c[7] << 16));
    }
    info[s] = it | (outside ? SLICE_SLOW_BIT : 0);
    if (outside) *outside_flag = 1;
}

// TH: the table holds fp16 rows (the strip is then 64 columns wide: a lane reads 16 bytes = eight columns of every row and
// sums them in fp32, native_kernels.cu:743-801 sparse_ft_forward_fp16); OH: the pre-activations are stored as fp16 and the
// activation is computed from the rounded value (sparse_ft_forward_fp16_out + ft_post_perspective_fwd_fp16, :837-863).
template <int MODE, bool TH, bool OH>
__global__ void __launch_bounds__(1024, 1) k_ft_forward_slice(const void* __restrict__ table_v, const float* __restrict__ bias,
                                                               void* __restrict__ pre_stm_v, void* __restrict__ pre_nstm_v,
                                                               float* __restrict__ combined, const int* __restrict__ idx_stm,
                                                               const int* __restrict__ idx_nstm, const int* __restrict__ info,
                                                               const uint4* __restrict__ codes, const FwdWork* __restrict__ work,
                                                               const int* __restrict__ n_work, int n_items, int B, int F, int N,
                                                               int A, int A_pad, int rps, float scale) {
    constexpr int W = TH ? 8 : 4;          // columns per lane
    constexpr int TSZ = TH ? 2 : 4;        // bytes per table element
    constexpr int OSZ = OH ? 2 : 4;        // bytes per stored pre-activation
    // strip [rps + 1][8 W] elements (128 bytes per row), then two buffers of [32 warps][4 items][A_pad] 16-bit row codes
    extern __shared__ __align__(16) unsigned char s_raw[];
    if ((int)blockIdx.x >= *n_work) return;
    const FwdWork wk = work[blockIdx.x];
    const int strip = blockIdx.y;
    const int row0 = wk.slice * rps;
    const int rows = max(0, min(rps, N - row0));
    const int half = F >> 1;
    const int cA = MODE == 1 ? 4 * W * strip : 8 * W * strip;  // first column of the strip's first half (or of all its columns)
    const int cB = MODE == 1 ? half + 4 * W * strip : cA + 4 * W;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 3, j = lane & 7;
    const int mycol = j < 4 ? cA + W * j : cB + W * (j - 4);
    const unsigned char* __restrict__ table = static_cast<const unsigned char*>(table_v);

    // strip fill: thread e & 7 == j copies the 16 bytes it will later read, for rows e >> 3
    for (int e = threadIdx.x; e < rows * 8; e += blockDim.x)
        cp_async16(s_raw + (size_t)e * 16, table + ((size_t)(row0 + (e >> 3)) * F + mycol) * TSZ, 16);
    if (threadIdx.x < 32) reinterpret_cast<float*>(s_raw)[rps * 32 + threadIdx.x] = 0.f;  // the row of zeros
    for (int e = rows * 8 + threadIdx.x; e < rps * 8; e += blockDim.x)  // rows past the end of the table
        *reinterpret_cast<float4*>(s_raw + (size_t)e * 16) = make_float4(0.f, 0.f, 0.f, 0.f);

    // a round = four items per warp; their codes arrive by asynchronous copy one round ahead
    const int code_bytes = 4 * A_pad * 2;  // per warp and buffer
    unsigned char* s_codes = s_raw + ((size_t)rps + 1) * 128 + (size_t)warp * code_bytes;
    const int buf_stride = 32 * code_bytes;
    const unsigned char* codes_b = reinterpret_cast<const unsigned char*>(codes);
    const int chunk_item = (lane * 16) / (A_pad * 2);  // which of the four items this lane's 16-byte piece belongs to
    auto fetch_codes = [&](int slot, int buf) {
        if (lane * 16 < code_bytes) {
            // pieces of slots past the end of the run are filled with zeros (row 0): whatever lies there is never a
            // valid offset into this block's strip
            const bool ok = slot + chunk_item < wk.end;
            const long long off = (long long)slot * A_pad * 2 + lane * 16;
            cp_async16(s_codes + buf * buf_stride + lane * 16, codes_b + (ok ? off : 0), ok ? 16 : 0);
        }
    };
    const int per_round = 4 * (blockDim.x >> 5);
    fetch_codes(wk.begin + 4 * warp, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // fp32 lanes keep the bias of their four columns and of the pair partner's in registers; fp16 lanes (eight columns)
    // read it in the epilogue instead (L1 hits), their registers are taken by the wider running sums
    float4 mybias = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!TH && bias) mybias = *reinterpret_cast<const float4*>(bias + mycol);
    float4 pbias = mybias;  // the pair partner's bias (LayerStack)
    pbias.x = __shfl_xor_sync(0xffffffffu, mybias.x, 4); pbias.y = __shfl_xor_sync(0xffffffffu, mybias.y, 4);
    pbias.z = __shfl_xor_sync(0xffffffffu, mybias.z, 4); pbias.w = __shfl_xor_sync(0xffffffffu, mybias.w, 4);
    const unsigned char* s_lane = s_raw + 16 * j;

    int buf = 0;
    for (int base = wk.begin; base < wk.end; base += per_round, buf ^= 1) {
        const int slot = base + 4 * warp + g;
        const int inf = slot < wk.end ? __ldg(info + slot) : -1;
        fetch_codes(base + per_round + 4 * warp, buf ^ 1);  // the other buffer was last read a round ago (warp barrier below)
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const bool slow = __any_sync(0xffffffffu, inf >= 0 && (inf & SLICE_SLOW_BIT));
        const int it_c = inf < 0 ? -1 : (inf & ~SLICE_SLOW_BIT);
        const unsigned char* my_codes = s_codes + buf * buf_stride + g * A_pad * 2;

        LaneAcc<TH> acc;
        acc.zero();
        if (!slow) {
            // every row of the round comes from the strip: branch-free; a slot without a feature reads the row of zeros
            // (x + 0.0 == x), rows are added in slot order
#pragma unroll 1
            for (int q = 0; q < A_pad; q += 8) {
                const uint4 c = *reinterpret_cast<const uint4*>(my_codes + 2 * q);
                const ulonglong2 v0 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.x & 0xffffu) * 128u);
                const ulonglong2 v1 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.x >> 16) * 128u);
                const ulonglong2 v2 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.y & 0xffffu) * 128u);
                const ulonglong2 v3 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.y >> 16) * 128u);
                const ulonglong2 v4 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.z & 0xffffu) * 128u);
                const ulonglong2 v5 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.z >> 16) * 128u);
                const ulonglong2 v6 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.w & 0xffffu) * 128u);
                const ulonglong2 v7 = *reinterpret_cast<const ulonglong2*>(s_lane + (c.w >> 16) * 128u);
                acc.add(v0); acc.add(v1); acc.add(v2); acc.add(v3);
                acc.add(v4); acc.add(v5); acc.add(v6); acc.add(v7);
            }
        } else {
            const int p = it_c >= B, bb = it_c < 0 ? 0 : it_c - p * B;
            const int* ip = (p ? idx_nstm : idx_stm) + (size_t)bb * A;
            for (int q = 0; q < A_pad; ++q) {
                const unsigned c = reinterpret_cast<const unsigned short*>(my_codes)[q];
                ulonglong2 v;
                if (c != SLICE_OUTSIDE || it_c < 0) v = *reinterpret_cast<const ulonglong2*>(s_lane + min(c, (unsigned)rps) * 128u);
                else v = __ldg(reinterpret_cast<const ulonglong2*>(table + ((size_t)__ldg(ip + q) * F + mycol) * TSZ));
                acc.add(v);
            }
        }
        __syncwarp();  // all lanes are done with this round's codes before the next round overwrites the other buffer's twin

        // ---- epilogue: x[] = the lane's sums as the later kernels will read them (rounded to fp16 when stored so)
        float x[W];
#pragma unroll
        for (int i = 0; i < W; ++i) x[i] = acc.get(i);
        const bool valid = it_c >= 0;
        const int persp = it_c >= B, b = valid ? it_c - persp * B : 0;
        unsigned char* pre = static_cast<unsigned char*>(persp ? pre_nstm_v : pre_stm_v) + ((size_t)b * F + mycol) * OSZ;
        auto store_pre = [&](const float* val) {
            if (OH) {
                unsigned h[W / 2];
#pragma unroll
                for (int i = 0; i < W / 2; ++i) h[i] = pack_h2(val[2 * i], val[2 * i + 1]);
                if (W == 8) __stcs(reinterpret_cast<uint4*>(pre), make_uint4(h[0], h[1], h[W / 2 - 2], h[W / 2 - 1]));
                else __stcs(reinterpret_cast<uint2*>(pre), make_uint2(h[0], h[1]));
            } else {
#pragma unroll
                for (int i = 0; i < W; i += 4) __stcs(reinterpret_cast<float4*>(pre) + i / 4, make_float4(val[i], val[i + 1], val[i + 2], val[i + 3]));
            }
        };
        if (OH) {
#pragma unroll
            for (int i = 0; i < W; i += 2) {
                const float2 r = unpack_h2(pack_h2(x[i], x[i + 1]));
                x[i] = r.x; x[i + 1] = r.y;
            }
        }
        if (MODE == 0) {
            if (valid) store_pre(x);
        } else if (MODE == 1) {
            float px[W];  // the pair partner's values
#pragma unroll
            for (int i = 0; i < W; ++i) px[i] = __shfl_xor_sync(0xffffffffu, x[i], 4);
            if (valid) {
                store_pre(x);
                if (j < 4) {
                    float o[W], bm[W], bp[W];
                    if (TH) {
#pragma unroll
                        for (int i = 0; i < W; i += 4) {
                            const float4 u = __ldg(reinterpret_cast<const float4*>(bias + mycol + i));
                            const float4 w = __ldg(reinterpret_cast<const float4*>(bias + half + mycol + i));
                            bm[i] = u.x; bm[i + 1] = u.y; bm[i + 2] = u.z; bm[i + 3] = u.w;
                            bp[i] = w.x; bp[i + 1] = w.y; bp[i + 2] = w.z; bp[i + 3] = w.w;
                        }
                    } else {
                        bm[0] = mybias.x; bm[1] = mybias.y; bm[2] = mybias.z; bm[3] = mybias.w;
                        bp[0] = pbias.x; bp[1] = pbias.y; bp[2] = pbias.z; bp[3] = pbias.w;
                    }
#pragma unroll
                    for (int i = 0; i < W; ++i) o[i] = crelu01(x[i] + bm[i]) * crelu01(px[i] + bp[i]) * scale;
                    float4* dst = reinterpret_cast<float4*>(combined + (size_t)b * F + persp * half + mycol);
#pragma unroll
                    for (int i = 0; i < W; i += 4) __stcs(dst + i / 4, make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]));
                }
            }
        } else if (valid) {
            float y[W], a[W];
            const float bz[4] = {mybias.x, mybias.y, mybias.z, mybias.w};
#pragma unroll
            for (int i = 0; i < W; ++i) {
                y[i] = x[i] + (TH ? __ldg(bias + mycol + i) : bz[i & 3]);
                a[i] = crelu01(y[i]);
                if (MODE == 3) a[i] *= a[i];
            }
            store_pre(y);
            float4* dst = reinterpret_cast<float4*>(combined + (size_t)b * 2 * F + persp * F + mycol);
#pragma unroll
            for (int i = 0; i < W; i += 4) __stcs(dst + i / 4, make_float4(a[i], a[i + 1], a[i + 2], a[i + 3]));
        }
    }
    cp_async_wait<0>();  // nothing of this block is in flight when it leaves
}


// work: FwdWork records, one int (their count), the slot info [n_items], then the 16-bit row codes [n_items][A rounded up to 8]
size_t ft_forward_slice_work_ints(int n_items, int n_keys, int A) {
    return 4 * slice_max_work(n_items, n_keys) + 4 + ((size_t)n_items + 3) / 4 * 4 + ((size_t)n_items * slice_a_pad(A) + 1) / 2 + 4;
}

static inline size_t slice_smem_bytes(int rps, int A) { return ((size_t)rps + 1) * 128 + (size_t)2 * 32 * 4 * slice_a_pad(A) * 2; }

bool ft_forward_slice_supported(int F, int N, int A, int rps) {
    int n_slices = ceil_div(N, rps);
    return F % 128 == 0 && A <= 64 && rps < 0xFFFF && slice_smem_bytes(rps, A) <= 227 * 1024 && n_slices + 1 <= SORT_KEYS_MAX;
}

int launch_ft_forward_slice(cudaStream_t s, int mode, const void* table, const int* idx_stm, const int* idx_nstm,
                            const int* nnz, const float* bias, void* pre_stm, void* pre_nstm, float* combined,
                            const int* items, const int* item_seg, int* work, int B, int F, int N, int A, int rps,
                            float scale, int n_persp, int table_half, int out_half) {
    if (B <= 0) return 0;
    const int n_items = n_persp * B;
    const int n_slices = ceil_div(N, rps), n_keys = n_slices + 1;
    const int max_work = (int)slice_max_work(n_items, n_keys);
    const int A_pad = slice_a_pad(A);
    const SliceBuffers sb = slice_buffers(work, n_items, n_keys);
    FwdWork* wk = sb.work;
    int* n_work = sb.n_work;
    int* info = sb.info;
    uint4* codes = sb.codes;
    k_fwd_plan<<<1, 128, 0, s>>>(item_seg, n_keys, SLICE_IPC, wk, n_work);
    k_fwd_codes<<<ceil_div(n_items, 256), 256, 0, s>>>(idx_stm, idx_nstm, nnz, items, item_seg, n_keys, n_items, B, N, A, A_pad,
                                                       rps, codes, info, sb.outside_flag);
    const size_t smem = slice_smem_bytes(rps, A);
    dim3 grid(max_work, table_half ? F / 64 : F / 32);
#define FT_SLICE_LAUNCH(M, TH, OH)                                                                                       \
    do {                                                                                                                 \
        cudaFuncSetAttribute(k_ft_forward_slice<M, TH, OH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        k_ft_forward_slice<M, TH, OH><<<grid, 1024, smem, s>>>(table, bias, pre_stm, pre_nstm, combined, idx_stm, idx_nstm, \
                                                               info, codes, wk, n_work, n_items, B, F, N, A, A_pad, rps, \
                                                               scale);                                                   \
    } while (0)
    if (table_half) {  // fp16 table: the raw gather (mode 0) and the LayerStack activation, with fp32 or fp16 pre-activations
        if (mode == 0 && !out_half) FT_SLICE_LAUNCH(0, true, false);
        else if (mode == 1 && !out_half) FT_SLICE_LAUNCH(1, true, false);
        else if (mode == 1) FT_SLICE_LAUNCH(1, true, true);
        else return -1;
    } else {
        if (out_half) return -1;
        switch (mode) {
            case 0: FT_SLICE_LAUNCH(0, false, false); break;
            case 1: FT_SLICE_LAUNCH(1, false, false); break;
            case 2: FT_SLICE_LAUNCH(2, false, false); break;
            default: FT_SLICE_LAUNCH(3, false, false); break;
        }
    }
#undef FT_SLICE_LAUNCH
    return 3;
}

// ------------------------------------------------------------------------------------------------
// inverse index: for every feature the list of positions that hold it (the counting sort of
// native_kernels.cu:1630-1765: histogram, exclusive scan, ranked scatter).
// ------------------------------------------------------------------------------------------------
__global__ void k_feat_count(const int* __restrict__ idx_stm, const int* __restrict__ idx_nstm,
                             const int* __restrict__ nnz, int B, int A, int N, int n_persp, int* __restrict__ counts, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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
                                                           int* __restrict__ block_sums, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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
                                                         const int* __restrict__ block_sums, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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
                            int* __restrict__ lists, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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
// Short lists (<= 32 * SORT_WARP_VALUES = 256 entries): one warp ranks its entries against each other through shuffles.
// Long lists: queued, then one block per list marks the positions in a shared-memory bitmap and reads
// the set bits back in order; a list that names a position twice (only possible when the caller's
// index row repeats a feature) falls back to ranking by counting.
#define SORT_WARP_VALUES 8  // list entries a lane holds in the warp-level sort
// one warp sorts L[0 .. len), len <= 32 V: lane l holds entries l, l + 32, ..; every entry is ranked against all entries of
// the list (ties by index: the bitmap kernel's fallback treats repeated positions the same way)
template <int V>
static __device__ __forceinline__ void warp_rank_sort(int* __restrict__ L, int len, int lane) {
    int v[V], r[V];
#pragma unroll
    for (int m = 0; m < V; ++m) {
        v[m] = lane + 32 * m < len ? L[lane + 32 * m] : 0x7fffffff;
        r[m] = 0;
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
        if (32 * k >= len) break;  // uniform over the warp
        const int nj = min(32, len - 32 * k);
        for (int l = 0; l < nj; ++l) {
            const int u = __shfl_sync(0xffffffffu, v[k], l);
            const int j = 32 * k + l;
#pragma unroll
            for (int m = 0; m < V; ++m) r[m] += (u < v[m]) || (u == v[m] && j < lane + 32 * m);
        }
    }
    __syncwarp();
#pragma unroll
    for (int m = 0; m < V; ++m)
        if (lane + 32 * m < len) L[r[m]] = v[m];
}

__global__ void __launch_bounds__(256) k_lists_sort_short(const int* __restrict__ offsets, int N, int n_persp, int B, int A,
                                                           int* __restrict__ lists, int* __restrict__ long_queue,
                                                           int* __restrict__ long_count, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
    const int lane = threadIdx.x & 31;
    for (int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; warp < n_persp * N; warp += (gridDim.x * blockDim.x) >> 5) {
    const int p = warp / N, f = warp - p * N;
    const int beg = offsets[(size_t)p * (N + 1) + f], end = offsets[(size_t)p * (N + 1) + f + 1];
    const int len = end - beg;
    if (len < 2) continue;
    if (len > 32 * SORT_WARP_VALUES) {
        if (lane == 0) long_queue[atomicAdd(long_count, 1)] = warp;
        continue;
    }
    int* L = lists + (size_t)p * B * A + beg;
    if (len <= 64) warp_rank_sort<2>(L, len, lane);
    else warp_rank_sort<SORT_WARP_VALUES>(L, len, lane);
    }
}

__global__ void __launch_bounds__(256) k_lists_sort_long(const int* __restrict__ offsets, int N, int B, int A,
                                                          int* __restrict__ lists, int* __restrict__ scratch,
                                                          const int* __restrict__ long_queue,
                                                          const int* __restrict__ long_count, int bitmap_words, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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

int launch_inverse_index(cudaStream_t s, const int* run_if, const int* idx_stm, const int* idx_nstm, const int* nnz, int B, int A,
                         int N, int n_persp, int* counts, int* offsets, int* cursor, int* lists) {
    if (B <= 0) return 0;
    // counts holds [2][N] histogram cells followed by one counter and a queue of [2*N] long-list ids
    int* long_count = counts + (size_t)2 * N;
    int* long_queue = long_count + 1;
    cudaMemsetAsync(counts, 0, sizeof(int) * ((size_t)2 * N + 1), s);
    const long long total = (long long)n_persp * B * A;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    k_feat_count<<<blocks, 256, 0, s>>>(idx_stm, idx_nstm, nnz, B, A, N, n_persp, counts, run_if);
    {   // block sums live behind the long-list queue (which holds at most 2N ids)
        int* block_sums = long_queue + (size_t)2 * N;
        const dim3 sg(ceil_div(N, SCAN_CELLS), n_persp);
        k_feat_scan_local<<<sg, 1024, 0, s>>>(counts, N, offsets, block_sums, run_if);
        k_feat_scan_add<<<sg, 1024, 0, s>>>(N, offsets, cursor, block_sums, run_if);
    }
    k_feat_fill<<<blocks, 256, 0, s>>>(idx_stm, idx_nstm, nnz, B, A, N, n_persp, cursor, lists, run_if);
    int* scratch = lists + (size_t)2 * B * A;  // the list buffer carries a second copy's worth of room
    const long long warps = (long long)n_persp * N;
    k_lists_sort_short<<<(int)(run_if && (warps * 32 + 255) / 256 > 148 * 32 ? 148 * 32 : (warps * 32 + 255) / 256), 256, 0, s>>>(offsets, N, n_persp, B, A, lists, long_queue, long_count, run_if);
    int words = (B + 31) / 32;
    if ((size_t)words * 4 > 160 * 1024) words = 0;
    // per device and cheap: set before every launch (a process may drive several GPUs)
    cudaFuncSetAttribute(k_lists_sort_long, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    k_lists_sort_long<<<148 * 4, 256, (size_t)words * 4, s>>>(offsets, N, B, A, lists, scratch, long_queue, long_count, words, run_if);
    return 6;
}

// ------------------------------------------------------------------------------------------------
// backward: a block per feature row, a thread per float4 column.  The row of the gradient is written exactly once per
// step (stm list first, then nstm list, each in ascending position order: the accumulation order of
// sparse_ft_backward_cpu called for stm then nstm), with list splitting: a feature that is active in very many positions (the king square of a
// king bucket, a pawn in hand) makes one block walk a list of thousands of rows; with real, skewed data such
// lists reach tens of thousands of entries and would set the kernel's run time on their own.  Features whose
// lists (stm + nstm) exceed BWD_PART entries are cut into parts of BWD_PART entries; every part is summed
// by its own block into a scratch row, and a last kernel adds the parts of a feature in order.  Which
// block gets which part depends on timing, the sums do not.
// ------------------------------------------------------------------------------------------------
#define BWD_PART 4096

__global__ void k_bwd_plan(const int* __restrict__ offsets, int N, int n_persp, int* __restrict__ counters,
                           int2* __restrict__ work, int* __restrict__ longf, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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

template <bool DH>
static __device__ __forceinline__ float4 sum_rows(const void* __restrict__ d, const int* __restrict__ L, int beg, int end,
                                                  int F, int c, float4 acc) {
    for (int j = beg; j < end; j += 8) {
        int bi[8];
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) bi[u] = __ldg(L + min(j + u, end - 1));
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = ld4<DH>(d, (size_t)bi[u] * F + 4 * c);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (j + u < end) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
        }
    }
    return acc;
}

// DH: the incoming gradient rows are fp16 (summed in fp32, native_kernels.cu:1081-1140); the sums are then left in the
// rows' loss scale, which the optimizer takes out again
template <bool DH>
__global__ void __launch_bounds__(512) k_ft_backward_short(const void* __restrict__ dft_stm, const void* __restrict__ dft_nstm,
                                                             const int* __restrict__ offsets, const int* __restrict__ lists,
                                                             int B, int A, int N, int F, int n_persp, float* __restrict__ grad, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int row4 = F >> 2;
    for (int f = blockIdx.x; f < N; f += gridDim.x) {
    int len = offsets[f + 1] - offsets[f];
    if (n_persp > 1) len += offsets[(size_t)(N + 1) + f + 1] - offsets[(size_t)(N + 1) + f];
    if (len > BWD_PART) continue;  // summed in parts by k_ft_backward_long
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < n_persp; ++p) {
        const int beg = offsets[(size_t)p * (N + 1) + f], end = offsets[(size_t)p * (N + 1) + f + 1];
        // unconditional loads (a slot past the end re-reads the last row and is dropped), so that all eight row loads
        // are in flight together
        acc = sum_rows<DH>(p ? dft_nstm : dft_stm, lists + (size_t)p * B * A, beg, end, F, c, acc);
    }
    reinterpret_cast<float4*>(grad)[(size_t)f * row4 + c] = acc;
    }
}

template <bool DH>
__global__ void __launch_bounds__(512) k_ft_backward_long(const void* __restrict__ dft_stm, const void* __restrict__ dft_nstm,
                                                            const int* __restrict__ offsets, const int* __restrict__ lists,
                                                            int B, int A, int N, int F, int n_persp,
                                                            const int* __restrict__ counters, const int2* __restrict__ work,
                                                            float* __restrict__ partial, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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
                acc = sum_rows<DH>(p ? dft_nstm : dft_stm, lists + (size_t)p * B * A, beg + a, beg + b, F, c, acc);
            lo -= len;
            hi -= len;
        }
        reinterpret_cast<float4*>(partial)[(size_t)w * row4 + c] = acc;
    }
}

__global__ void __launch_bounds__(512) k_ft_backward_long_final(const int* __restrict__ counters, const int* __restrict__ longf,
                                                                  const float* __restrict__ partial, int F,
                                                                  float* __restrict__ grad, const int* __restrict__ run_if) {
    if (run_if && *run_if == 0) return;  // gated: another path does this step's work
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
int launch_ft_backward_split(cudaStream_t s, const int* run_if, const void* dft_stm, const void* dft_nstm, const int* offsets,
                             const int* lists, int B, int A, int N, int F, int n_persp, int* plan, float* partial,
                             float* grad, int dft_half) {
    const int max_work = ft_backward_max_work(B, A, n_persp);
    int* counters = plan;
    int2* work = reinterpret_cast<int2*>(plan + 2);
    int* longf = plan + 2 + 2 * max_work;
    cudaMemsetAsync(counters, 0, 2 * sizeof(int), s);
    k_bwd_plan<<<ceil_div(N, 256), 256, 0, s>>>(offsets, N, n_persp, counters, work, longf, run_if);
    const int ny = ceil_div(F / 4, 512), bx = F / 4 / ny;  // at most 512 threads per block: room for 64 registers each
    // a gated launch (run_if) normally returns at once: a small grid of row-striding blocks keeps that cheap
    const dim3 gs(run_if && N > 148 * 32 ? 148 * 32 : N, ny), gl(148 * 4, ny);
    if (dft_half) {
        k_ft_backward_short<true><<<gs, bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, grad, run_if);
        k_ft_backward_long<true><<<gl, bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, counters, work, partial, run_if);
    } else {
        k_ft_backward_short<false><<<gs, bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, grad, run_if);
        k_ft_backward_long<false><<<gl, bx, 0, s>>>(dft_stm, dft_nstm, offsets, lists, B, A, N, F, n_persp, counters, work, partial, run_if);
    }
    k_ft_backward_long_final<<<dim3(148 * 2, ny), bx, 0, s>>>(counters, longf, partial, F, grad, run_if);
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

// ft_fold_virtual (sparse/ft_factorize.rs:78-99): comb[f] = w[f] + w[N + f % pi]; HC: rounded to fp16
// (ft_fold_virtual_f16, native_kernels.cu:262-318)
template <bool HC>
__global__ void k_ft_fold(const float* __restrict__ w, void* __restrict__ comb, int N, int pi, int F) {
    const int row4 = F >> 2;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)N * row4) return;
    const int f = (int)(i / row4), c = (int)(i - (long long)f * row4);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const float4 a = w4[i];
    const float4 b = w4[(size_t)(N + f % pi) * row4 + c];
    const float4 v = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
    if (HC) static_cast<uint2*>(comb)[i] = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
    else static_cast<float4*>(comb)[i] = v;
}

int launch_ft_fold(cudaStream_t s, const float* w, void* comb, int N, int pi, int F, int half_comb) {
    const long long n = (long long)N * (F / 4);
    if (half_comb) k_ft_fold<true><<<(int)((n + 255) / 256), 256, 0, s>>>(w, comb, N, pi, F);
    else k_ft_fold<false><<<(int)((n + 255) / 256), 256, 0, s>>>(w, comb, N, pi, F);
    return 1;
}

// cast_f32_to_f16 (native_kernels.cu:648): the fp16 mirror of an fp32 table
__global__ void k_cast_half(const float4* __restrict__ src, uint2* __restrict__ dst, long long n4) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const float4 v = src[i];
        dst[i] = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
    }
}

int launch_cast_half(cudaStream_t s, const float* src, void* dst, int64_t n) {
    const long long n4 = n / 4;
    long long blocks = (n4 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    k_cast_half<<<(int)blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(src), static_cast<uint2*>(dst), n4);
    return 1;
}
