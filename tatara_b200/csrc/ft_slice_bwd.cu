// FT weight gradient, slice-resident variant (the transposed twin of k_ft_forward_slice).
//
// When every feature of an item lies in the item's own king-bucket slice of the table (true for the king-relative
// feature sets by construction; k_fwd_codes checks it for the batch at hand), a feature row of slice k is touched
// only by the items sorted into slice k.  The slice's items are cut into chunks of <= CH consecutive slots; for
// each chunk one block builds the inverse index locally (k_inv_chunk: for every row of the slice the ascending
// list of chunk-local slots that hold it, by a counting sort in shared memory whose integer atomics only hand out
// ranks inside one slot, so the lists come out ascending without a per-list sort), and the gradient kernel keeps a 32-column strip of the chunk's dft rows in shared memory together with
// all of the chunk's lists, so that every row read of the sum comes from shared memory.
// A block owns (slice, column strip), walks the slice's chunks in order and carries the running sums through the
// gradient rows themselves, so a row's terms are added one by one in ascending item order: the result is
// bit-identical to the per-row sequential sum of the generic kernels (stm items first, ascending position).
// Exception: a list with BWD_HOT or more entries inside one chunk is summed there as four partial sums (its
// quarters in order), combined as prev + ((p0 + p1) + (p2 + p3)): a fixed order as well, so results stay
// reproducible run to run, but not the sequential one.  (The reference's own kernel keeps four interleaved partial
// sums over a list whose order is set by atomics, native_kernels.cu:1767-1806.)
//
// Skewed data (real king squares crowd a few buckets): a slice's chunks are handed out in groups of BWD_GROUP consecutive
// chunks, a block per (group, column strip), so that a slice holding a third of the batch does not leave its strips'
// blocks running alone.  The first group of a slice writes the gradient rows, every further group a partial slab of its
// own, and k_bwd_combine adds the slabs onto the rows in group order: one more fixed, non-sequential association, used
// only by slices of more than BWD_GROUP chunks (about 3600 items).
//
// Both kernels return at once when the batch has a row outside its item's slice (outside_flag != 0); the generic
// kernels, gated the other way round, then do the work.
#include "ft_slice.cuh"

#define INV_SORT_N 2048  // rows per slice limit (bitonic sort size)
#define BWD_HOT 256      // list length from which a list is summed as four quarters by the four groups of one warp
#define BWD_DESC 64      // chunk descriptors a block stages in shared memory
#define BWD_GROUP 4      // chunks per block: a slice of more chunks is shared by several blocks

struct BwdLayout {
    int CH;             // slots per chunk (multiple of 8)
    int rps_pad;        // row records per chunk
    int region;         // 16-bit list cells per chunk (every list is padded to a multiple of 8 cells: 16-byte code loads)
    int max_chunks;
    int max_groups, max_slabs;  // (slice, chunk group) work units; partial slabs of the groups behind a slice's first
    size_t off_first, off_len, off_groups, off_rowinfo, off_lists, total_ints;
};

static inline size_t bwd_region(int CH, int rps, int A_pad) { return (size_t)CH * A_pad + 8 * (size_t)rps; }

static inline size_t bwd_smem_bytes(int CH, int rps, int A_pad) {
    const int rps_pad = (rps + 3) / 4 * 4;
    return ((size_t)CH + 1) * 128 + (size_t)rps_pad * 8 + bwd_region(CH, rps, A_pad) * 2;
}

static inline BwdLayout bwd_layout(int n_items, int A, int rps) {
    BwdLayout L;
    const int A_pad = slice_a_pad(A);
    int CH = 0;
    for (int c = 32; c <= 4096; c += 8) {
        if (bwd_smem_bytes(c, rps, A_pad) + 2048 > 227 * 1024) break;  // 2 KB stay free for the kernels' static arrays
        if (bwd_region(c, rps, A_pad) > 65535) break;
        // k_inv_chunk: histograms, offsets and sort keys, the chunk's lists
        if ((size_t)64 * ((rps + 1) & ~1) + (size_t)INV_SORT_N * 8 + bwd_region(c, rps, A_pad) * 2 + 2048 > 227 * 1024) break;
        CH = c;
    }
    L.CH = CH;
    L.rps_pad = (rps + 3) / 4 * 4;
    L.region = (int)bwd_region(CH, rps, A_pad);
    L.max_chunks = CH > 0 ? n_items / CH + SORT_KEYS_LIMIT + 2 : 0;
    L.max_slabs = CH > 0 ? n_items / (CH * BWD_GROUP) + SORT_KEYS_LIMIT / BWD_GROUP + 2 : 0;
    L.max_groups = SORT_KEYS_LIMIT + L.max_slabs;
    size_t o = 4 * (size_t)L.max_chunks + 4;            // chunk records + their count
    L.off_first = o; o += SORT_KEYS_LIMIT + 4;          // first chunk of every slice (+ end)
    L.off_len = o; o += 4 * (size_t)L.max_chunks;  // per chunk {list cells, long-list records, non-empty records, 0}
    // groups: [0] their count, [4 ..] first group of every slice (+ end), then {slice, first chunk, end chunk, slab or -1}
    L.off_groups = o; o += 4 + (SORT_KEYS_LIMIT + 4) + 4 * (size_t)L.max_groups;
    L.off_rowinfo = o; o += 2 * (size_t)L.max_chunks * L.rps_pad;
    L.off_lists = o; o += ((size_t)L.max_chunks * L.region + 1) / 2 + 4;
    L.total_ints = o;
    return L;
}

bool ft_backward_slice_supported(int F, int N, int A, int rps) {
    const int n_slices = ceil_div(N, rps);
    if (!(F % 128 == 0 && A <= 64 && rps <= INV_SORT_N && n_slices + 1 <= SORT_KEYS_LIMIT)) return false;
    return bwd_layout(1024, A, rps).CH >= 64;
}

size_t ft_backward_slice_ints(int n_items, int A, int rps) { return bwd_layout(n_items, A, rps).total_ints; }
size_t ft_backward_slice_slab_floats(int n_items, int A, int rps, int F) {
    return (size_t)bwd_layout(n_items, A, rps).max_slabs * (size_t)rps * (size_t)F;
}

// chunks of <= ipc consecutive slots of one slice; first[k] = index of slice k's first chunk, first[n_keys] = total
__global__ void k_chunk_plan(const int* __restrict__ item_seg, int n_keys, int ipc, FwdWork* __restrict__ work,
                             int* __restrict__ n_work, int* __restrict__ first, int* __restrict__ groups, int max_groups) {
    __shared__ int s_base[SORT_KEYS_LIMIT + 1], s_seg[SORT_KEYS_LIMIT + 2];
    for (int k = threadIdx.x; k <= n_keys; k += blockDim.x) s_seg[k] = item_seg[k];  // one round trip, not n_keys
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int k = 0; k < n_keys; ++k) {
            s_base[k] = run;
            run += (s_seg[k + 1] - s_seg[k] + ipc - 1) / ipc;
        }
        s_base[n_keys] = run;
        *n_work = run;
        // (slice, chunk group) work units of the real slices (the last key holds items without a slice: they have no rows)
        int* group_first = groups + 4;
        int4* rec = reinterpret_cast<int4*>(groups + 4 + SORT_KEYS_LIMIT + 4);
        int gi = 0, slab = 0;
        for (int k = 0; k < n_keys - 1; ++k) {
            group_first[k] = gi;
            const int c0 = s_base[k], nc = s_base[k + 1] - c0;
            if (nc == 0 && gi < max_groups) rec[gi++] = make_int4(k, c0, c0, -1);  // an empty slice: its rows are zeroed
            for (int c = 0; c < nc && gi < max_groups; c += BWD_GROUP) rec[gi++] = make_int4(k, c0 + c, c0 + min(nc, c + BWD_GROUP), c == 0 ? -1 : slab++);
        }
        group_first[n_keys - 1] = gi;
        groups[0] = gi;
    }
    __syncthreads();
    for (int k = threadIdx.x; k <= n_keys; k += blockDim.x) first[k] = s_base[k];
    for (int k = 0; k < n_keys; ++k) {
        const int b0 = s_seg[k], e0 = s_seg[k + 1];
        const int n = s_base[k + 1] - s_base[k];
        const int size = n > 0 ? ((e0 - b0 + n - 1) / n + 7) & ~7 : 0;  // equal chunks (<= ipc: ipc is a multiple of 8)
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

// Inverse index of one chunk.  Shared memory: hist [32 warps][rps_h] 16-bit cells, rowoff [rps] ints, sort keys
// [INV_SORT_N] ints, the chunk's lists [region] 16-bit cells (copied out at the end in 16-byte pieces).  Warp w owns
// a contiguous range of the chunk's slots and walks it slot by slot, so "warp, then slot" is ascending slot order.
// rowinfo (sorted by descending list length, so that the eight-lane groups of a warp get lists of similar length
// and the long lists start first): row << 32 | list offset << 16 | list length; lists are padded to a multiple of
// eight cells with the index of the chunk's row of zeros (CH).
__global__ void __launch_bounds__(1024) k_inv_chunk(const unsigned short* __restrict__ codes, const FwdWork* __restrict__ work,
                                                    const int* __restrict__ n_work, const int* __restrict__ outside_flag,
                                                    int n_slices, int A_pad, int rps, int rps_pad, int CH, int region,
                                                    unsigned short* __restrict__ lists, unsigned long long* __restrict__ rowinfo,
                                                    int* __restrict__ len) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    if ((int)blockIdx.x >= *n_work || *outside_flag) return;
    const FwdWork wk = work[blockIdx.x];
    if (wk.slice >= n_slices) return;  // items without a slice have no rows
    const int rps_h = (rps + 1) & ~1;
    unsigned short* s_hist = reinterpret_cast<unsigned short*>(s_raw);                    // [32][rps_h]
    int* s_rowoff = reinterpret_cast<int*>(s_raw + (size_t)32 * rps_h * 2);               // [rps]
    unsigned* s_keys = reinterpret_cast<unsigned*>(s_rowoff + INV_SORT_N);                // [INV_SORT_N]
    unsigned short* s_lists = reinterpret_cast<unsigned short*>(s_keys + INV_SORT_N);     // [region]: the chunk's lists
    __shared__ int s_warp[32], s_total;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int n = wk.end - wk.begin;
    for (int e = tid; e < 16 * rps_h; e += 1024) reinterpret_cast<unsigned*>(s_hist)[e] = 0u;
    __syncthreads();

    const int per = (n + 31) >> 5;
    const int s0 = min(n, w * per), s1 = min(n, s0 + per);
    const int n_e = (s1 - s0) * A_pad;
    const unsigned short* cw = codes + (size_t)(wk.begin + s0) * A_pad;  // the warp's cells, consecutive in global memory
    unsigned short* my_hist = s_hist + (size_t)w * rps_h;

    // pass 1: per-warp histogram (two 16-bit cells per shared-memory word, bumped by 32-bit atomics; a cell never
    // reaches 65536, so no carry crosses into its neighbour)
    unsigned* my_hist32 = reinterpret_cast<unsigned*>(my_hist);
    for (int e0 = lane; e0 < n_e; e0 += 8 * 32) {  // eight loads in flight, then their atomics
        unsigned code[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) code[u] = e0 + 32 * u < n_e ? cw[e0 + 32 * u] : 0xFFFFu;
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (code[u] < (unsigned)rps) atomicAdd(my_hist32 + (code[u] >> 1), 1u << ((code[u] & 1u) * 16u));
    }
    __syncthreads();

    // per row: counts of the warps -> exclusive prefix over the warps; list offsets by a block scan of padded lengths
    const int rpt = (rps + 1023) >> 10;  // rows per thread (<= 2)
    int cnt[2] = {0, 0}, padded = 0;
    for (int u = 0; u < rpt; ++u) {
        const int r = tid * rpt + u;
        if (r < rps) {
            int run = 0;
            for (int ww = 0; ww < 32; ++ww) {
                const int c = s_hist[(size_t)ww * rps_h + r];
                s_hist[(size_t)ww * rps_h + r] = (unsigned short)run;
                run += c;
            }
            cnt[u] = run;
            padded += (run + 7) & ~7;
        }
    }
    int incl = padded;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
    }
    if (lane == 31) s_warp[w] = incl;
    __syncthreads();
    if (w == 0) {
        const int t = s_warp[lane];
        int ti = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, ti, d);
            if (lane >= d) ti += u;
        }
        s_warp[lane] = ti - t;
    }
    __syncthreads();
    unsigned short* my_lists = s_lists;
    int base = s_warp[w] + incl - padded;
    for (int u = 0; u < rpt; ++u) {
        const int r = tid * rpt + u;
        if (r < rps) {
            s_rowoff[r] = base;
            const int pe = base + ((cnt[u] + 7) & ~7);
            for (int i = base + cnt[u]; i < pe; ++i) my_lists[i] = (unsigned short)CH;
            base = pe;
        }
    }
    if (tid == 1023) { len[4 * blockIdx.x] = base; s_total = base; }
    if (tid == 0) { len[4 * blockIdx.x + 1] = 0; len[4 * blockIdx.x + 2] = 0; len[4 * blockIdx.x + 3] = 0; }
    // sort keys: ascending (65535 - length) << 11 | row, unused cells last
    for (int i = tid; i < INV_SORT_N; i += 1024) s_keys[i] = 0xFFFFFFFFu;
    __syncthreads();
    for (int u = 0; u < rpt; ++u) {
        const int r = tid * rpt + u;
        if (r < rps) s_keys[r] = ((unsigned)(65535 - cnt[u]) << 11) | (unsigned)r;
    }
    __syncthreads();
    for (int k = 2; k <= INV_SORT_N; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            const int i = ((tid & ~(j - 1)) << 1) | (tid & (j - 1));
            const int p = i | j;
            const unsigned a = s_keys[i], b = s_keys[p];
            const bool up = (i & k) == 0;
            if ((a > b) == up) { s_keys[i] = b; s_keys[p] = a; }
            __syncthreads();
        }
    }
    // the sorted order starts with the long lists and ends with the empty ones: where each group ends
    for (int i = tid; i < rps; i += 1024) {
        const int ci = 65535 - (int)(s_keys[i] >> 11);
        const int cn = i + 1 < rps ? 65535 - (int)(s_keys[i + 1] >> 11) : -1;
        if (ci >= BWD_HOT && cn < BWD_HOT) len[4 * blockIdx.x + 1] = i + 1;
        if (ci > 0 && cn <= 0) len[4 * blockIdx.x + 2] = i + 1;
    }
    unsigned long long* my_info = rowinfo + (size_t)blockIdx.x * rps_pad;
    for (int i = tid; i < rps_pad; i += 1024) {
        unsigned long long v = 0ull;  // row 0, empty list (cells past rps are never used)
        if (i < rps) {
            const unsigned key = s_keys[i];
            const unsigned r = key & 2047u, c = 65535u - (key >> 11);
            v = ((unsigned long long)r << 32) | ((unsigned long long)(unsigned)s_rowoff[r] << 16) | c;
        }
        my_info[i] = v;
    }

    // pass 2: ranked scatter of the chunk-local slot numbers.  A warp walks its slots one after the other, the lanes
    // take the slot's cells; the atomic's return value is the cell's rank inside the row's list.  Slots are visited in
    // ascending order, so every list comes out ascending (two cells of one slot carry the same value: their order is
    // immaterial).
    // (A_pad <= 64: a lane holds at most two cells of a slot; the next slot's cells are fetched while this one is placed)
    const int q1 = lane + 32;
    unsigned c0 = 0xFFFFu, c1 = 0xFFFFu;
    if (s0 < s1) {
        c0 = lane < A_pad ? cw[lane] : 0xFFFFu;
        c1 = q1 < A_pad ? cw[q1] : 0xFFFFu;
    }
    for (int sl = s0; sl < s1; ++sl) {
        unsigned n0 = 0xFFFFu, n1 = 0xFFFFu;
        if (sl + 1 < s1) {
            const unsigned short* nx = cw + (size_t)(sl + 1 - s0) * A_pad;
            n0 = lane < A_pad ? nx[lane] : 0xFFFFu;
            n1 = q1 < A_pad ? nx[q1] : 0xFFFFu;
        }
#pragma unroll
        for (int hq = 0; hq < 2; ++hq) {
            const unsigned code = hq ? c1 : c0;
            if (code < (unsigned)rps) {
                const unsigned sh = (code & 1u) * 16u;
                const unsigned old = atomicAdd(my_hist32 + (code >> 1), 1u << sh);
                my_lists[s_rowoff[code] + ((old >> sh) & 0xffffu)] = (unsigned short)sl;
            }
        }
        __syncwarp();
        c0 = n0; c1 = n1;
    }
    __syncthreads();
    // the finished lists leave in 16-byte pieces (the last piece may carry up to four cells nobody reads)
    {
        const int total = s_total;
        uint4* dst = reinterpret_cast<uint4*>(lists + (size_t)blockIdx.x * region);
        const uint4* src = reinterpret_cast<const uint4*>(s_lists);
        for (int e = tid; e < (total + 7) / 8; e += 1024) dst[e] = src[e];
    }
}

// grad[row][column strip] for the rows of one slice; see the head of the file.  DH: the dft rows are fp16 (the strip is
// then 64 columns wide, a lane sums eight columns in fp32; the sums keep the rows' loss scale).
template <bool DH>
__global__ void __launch_bounds__(1024, 1) k_ft_backward_slice(const void* __restrict__ dft_stm, const void* __restrict__ dft_nstm,
                                                                const int* __restrict__ info, const FwdWork* __restrict__ work,
                                                                const int* __restrict__ groups, const int* __restrict__ len,
                                                                const unsigned long long* __restrict__ rowinfo,
                                                                const unsigned short* __restrict__ lists,
                                                                const int* __restrict__ outside_flag, int B, int F, int N, int rps,
                                                                int rps_pad, int CH, int region, int slice_begin, int slice_count,
                                                                float* __restrict__ grad, float* __restrict__ slabs) {
    constexpr int W = DH ? 8 : 4;    // columns per lane
    constexpr int DSZ = DH ? 2 : 4;  // bytes per dft element
    typedef LaneAcc<DH> Acc;
    // dft strip [CH + 1][8 W] elements, 128 bytes per row (the last row stays zero), row records [rps_pad] 64-bit, list
    // cells [region] 16-bit
    extern __shared__ __align__(16) unsigned char s_raw[];
    __shared__ int s_ctl[4];
    __shared__ int s_desc[BWD_DESC][5];
    if (*outside_flag) return;
    // the groups of this launch's slices; the grid has a block row per slice, so a block takes a second group only when
    // some slice is shared (skewed data)
    // (the loop's state lives in shared memory: the body needs every register)
    __shared__ int s_gid;
    if (threadIdx.x == 0) s_gid = groups[4 + slice_begin] + (int)blockIdx.x;
    for (;;) {
    __syncthreads();  // s_gid written; the previous group's last reads of the shared buffers
    const int gid = s_gid;
    if (gid >= groups[4 + slice_begin + slice_count]) break;
    __syncthreads();  // every thread has read s_gid
    if (threadIdx.x == 0) s_gid = gid + (int)gridDim.x;
    const int4 gr = reinterpret_cast<const int4*>(groups + 4 + SORT_KEYS_LIMIT + 4)[gid];
    const int k = gr.x, strip = blockIdx.y;
    const int row0 = k * rps;
    const int rows = min(rps, N - row0);
    const int tid = threadIdx.x, lane = tid & 31;
    const int j = lane & 7;
    const int col = 8 * W * strip + W * j;
    const int c_first = gr.y, c_end = gr.z;
    // the slice's first group sums into the gradient rows, a later one into its own slab (combined by k_bwd_combine)
    float* __restrict__ out = gr.w < 0 ? grad + (size_t)row0 * F : slabs + (size_t)gr.w * rps * F;
    if (c_first == c_end) {  // no item reads this slice: its gradient rows are zero
        for (int e = tid; e < rows * 8; e += 1024) {
            float4* gp = reinterpret_cast<float4*>(out + (size_t)(e >> 3) * F + col);
#pragma unroll
            for (int i = 0; i < W / 4; ++i) gp[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        continue;
    }
    unsigned char* s_dft = s_raw;
    unsigned long long* s_info = reinterpret_cast<unsigned long long*>(s_raw + ((size_t)CH + 1) * 128);
    unsigned char* s_lists = reinterpret_cast<unsigned char*>(s_info + rps_pad);
    if (tid < 32) reinterpret_cast<float*>(s_dft)[CH * 32 + tid] = 0.f;
    const unsigned char* s_lane = s_dft + 16 * j;
    const unsigned char* __restrict__ d_stm = static_cast<const unsigned char*>(dft_stm);
    const unsigned char* __restrict__ d_nstm = static_cast<const unsigned char*>(dft_nstm);

    // the slice's chunk descriptors, fetched once (BWD_DESC at most; a slice with more chunks reads the rest as it goes)
    for (int i = tid; i < min(c_end - c_first, BWD_DESC); i += 1024) {
        const FwdWork wk = work[c_first + i];
        s_desc[i][0] = wk.begin; s_desc[i][1] = wk.end;
        s_desc[i][2] = len[4 * (c_first + i)]; s_desc[i][3] = len[4 * (c_first + i) + 1]; s_desc[i][4] = len[4 * (c_first + i) + 2];
    }
    __syncthreads();
    for (int c = c_first; c < c_end; ++c) {
        const int ci = c - c_first;
        const int wk_begin = ci < BWD_DESC ? s_desc[ci][0] : work[c].begin;
        const int wk_end = ci < BWD_DESC ? s_desc[ci][1] : work[c].end;
        const int n = wk_end - wk_begin;
        const int L = ci < BWD_DESC ? s_desc[ci][2] : len[4 * c];
        const int n_hot = ci < BWD_DESC ? s_desc[ci][3] : len[4 * c + 1];
        const int n_live = ci < BWD_DESC ? s_desc[ci][4] : len[4 * c + 2];
        __syncthreads();  // the previous chunk's sums are done with the buffers (and its gradient rows are written)
        {
            const unsigned char* src = reinterpret_cast<const unsigned char*>(rowinfo + (size_t)c * rps_pad);
            for (int e = tid; e < rps_pad / 2; e += 1024) cp_async16(reinterpret_cast<unsigned char*>(s_info) + (size_t)e * 16, src + (size_t)e * 16, 16);
            const unsigned char* lsrc = reinterpret_cast<const unsigned char*>(lists + (size_t)c * region);
            for (int e = tid; e < (L + 7) / 8; e += 1024) cp_async16(s_lists + (size_t)e * 16, lsrc + (size_t)e * 16, 16);
        }
        // dft rows: thread e & 7 == j copies the 16 bytes of row e >> 3 it will read.  The item numbers the addresses
        // depend on are fetched eight at a time before the copies, so that the copies go out back to back.
        for (int e0 = tid; e0 < n * 8; e0 += 8 * 1024) {
            int itv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = e0 + u * 1024;
                itv[u] = e < n * 8 ? __ldg(info + wk_begin + (e >> 3)) : 0;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = e0 + u * 1024;
                if (e < n * 8) {
                    const int it = itv[u] & ~SLICE_SLOW_BIT;
                    const int p = it >= B, b = it - p * B;
                    cp_async16(s_dft + (size_t)e * 16, (p ? d_nstm : d_stm) + ((size_t)b * F + col) * DSZ, 16);
                }
            }
        }
        if (tid == 0) s_ctl[1] = n_hot;  // the counter the records behind the long lists are handed out from
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        const bool first_chunk = c == c_first;
        // The records are sorted by descending list length.  A list of BWD_HOT entries or more gets a warp of its own,
        // whose four groups sum a quarter of it each: left to one group, its long chain of dependent additions would end
        // after the rest of the chunk.  All other records are handed out four at a time (neighbours in the order, so of
        // similar length) from a block-wide counter.
        const int n_rec = first_chunk ? rps : n_live;
        // sum of the list cells [beg, end) of one record, continuing from acc; beg is a multiple of 8.  Called by all
        // 32 lanes together (a group without a list passes an empty range)
        auto sum_range = [&](const unsigned char* lp, int beg, int end, Acc& acc) {
            const int full = beg + ((end - beg) & ~7);
            for (int q = beg; q < full; q += 8) {
                const uint4 cc = *reinterpret_cast<const uint4*>(lp + 2 * q);
                const ulonglong2 v0 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.x & 0xffffu) * 128u);
                const ulonglong2 v1 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.x >> 16) * 128u);
                const ulonglong2 v2 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.y & 0xffffu) * 128u);
                const ulonglong2 v3 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.y >> 16) * 128u);
                const ulonglong2 v4 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.z & 0xffffu) * 128u);
                const ulonglong2 v5 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.z >> 16) * 128u);
                const ulonglong2 v6 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.w & 0xffffu) * 128u);
                const ulonglong2 v7 = *reinterpret_cast<const ulonglong2*>(s_lane + (cc.w >> 16) * 128u);
                acc.add(v0); acc.add(v1); acc.add(v2); acc.add(v3);
                acc.add(v4); acc.add(v5); acc.add(v6); acc.add(v7);
            }
            // the last one to seven entries (the padding cells behind them are not read as rows).  All lanes of the warp
            // come here together: the loop runs as far as the longest remainder of the warp's four lists, so that no
            // load instruction is issued that none of them needs (the kernel is bound by the number of shared-memory
            // load instructions, not by their width).
            const int rem = end - full;
            const int rem_w = __reduce_max_sync(0xffffffffu, rem);
            if (rem_w > 0) {
                const uint4 cc = *reinterpret_cast<const uint4*>(lp + 2 * (rem > 0 ? full : 0));
                const unsigned cell[8] = {cc.x & 0xffffu, cc.x >> 16, cc.y & 0xffffu, cc.y >> 16,
                                          cc.z & 0xffffu, cc.z >> 16, cc.w & 0xffffu, cc.w >> 16};
                const ulonglong2 zero2 = make_ulonglong2(0ull, 0ull);
#pragma unroll
                for (int h = 0; h < 8; h += 4) {  // two halves of up to four loads, then their additions
                    if (h >= rem_w) break;
                    ulonglong2 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        v[u] = zero2;
                        if (h + u < 7 && h + u < rem_w) {
                            if (h + u < rem) v[u] = *reinterpret_cast<const ulonglong2*>(s_lane + cell[h + u] * 128u);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (h + u < rem) acc.add(v[u]);
                }
            }
        };
        const int warp = tid >> 5, g = lane >> 3;
        // long lists: the warp's four groups sum a quarter of the list each, then prev + ((p0 + p1) + (p2 + p3))
        for (int h = warp; h < n_hot; h += 32) {
            const unsigned long long ri = s_info[h];
            const int r = (int)(ri >> 32), off = (int)((ri >> 16) & 0xffffu), cnt = (int)(ri & 0xffffu);
            if (r >= rows) continue;
            const int qlen = (((cnt + 3) >> 2) + 7) & ~7;
            Acc part;
            part.zero();
            sum_range(s_lists + 2 * off, min(cnt, g * qlen), min(cnt, (g + 1) * qlen), part);
            part.add(part.shfl_xor(8));
            part.add(part.shfl_xor(16));
            if (g == 0) {
                float* gp = out + (size_t)r * F + col;
                if (!first_chunk) {
                    Acc pv;
                    pv.load_cg(gp);
                    part.add_from(pv);
                }
                part.store_cg(gp);
            }
        }
        // all other lists: one group each, the terms added one by one onto the running sum.  The next record and its
        // running sum (a gradient row written by the previous chunk) are fetched while the current record is summed.
        auto grab = [&]() {
            int base = 0;
            if (lane == 0) base = atomicAdd(&s_ctl[1], 4);
            return __shfl_sync(0xffffffffu, base, 0);
        };
        auto fetch = [&](int base, unsigned long long& ri, Acc& prev) {
            ri = ~0ull;  // no record
            prev.zero();
            if (base + g < n_rec) {
                const unsigned long long x = s_info[base + g];
                if ((int)(x >> 32) < rows) {
                    ri = x;
                    if (!first_chunk) prev.load_cg(out + (size_t)(int)(x >> 32) * F + col);
                }
            }
        };
        int base = grab();
        unsigned long long ri;
        Acc prev;
        fetch(base, ri, prev);
        while (base < n_rec) {
            const int base_n = grab();
            unsigned long long ri_n;
            Acc prev_n;
            fetch(base_n, ri_n, prev_n);
            {
                const bool have = ri != ~0ull;
                const int r = (int)(ri >> 32), off = have ? (int)((ri >> 16) & 0xffffu) : 0, cnt = have ? (int)(ri & 0xffffu) : 0;
                sum_range(s_lists + 2 * off, 0, cnt, prev);
                if (have) prev.store_cg(out + (size_t)r * F + col);
            }
            base = base_n; ri = ri_n; prev = prev_n;
        }
    }
    }  // groups of this block
}

// grad rows of a slice += its groups' slabs, in group order
__global__ void __launch_bounds__(256) k_bwd_combine(const int* __restrict__ groups, const int* __restrict__ outside_flag,
                                                      const float4* __restrict__ slabs, float4* __restrict__ grad, int rps, int F,
                                                      int N, int slice_begin) {
    if (*outside_flag) return;
    const int k = slice_begin + blockIdx.y;
    const int* group_first = groups + 4;
    const int4* rec = reinterpret_cast<const int4*>(groups + 4 + SORT_KEYS_LIMIT + 4);
    const int g0 = group_first[k], g1 = group_first[k + 1];
    if (g1 - g0 <= 1) return;
    const int rows = min(rps, N - k * rps);
    const size_t n4 = (size_t)rows * F / 4, slab4 = (size_t)rps * F / 4;
    float4* dst = grad + (size_t)k * rps * F / 4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 a = dst[i];
        for (int g = g0 + 1; g < g1; ++g) {
            const float4 v = __ldcs(slabs + (size_t)rec[g].w * slab4 + i);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        dst[i] = a;
    }
}

struct BwdPointers {
    FwdWork* chunks;
    int *n_chunks, *first, *len, *groups;
    unsigned long long* rowinfo;
    unsigned short* lists;
};
static inline BwdPointers bwd_pointers(int* bwd_work, const BwdLayout& L) {
    BwdPointers p;
    p.chunks = reinterpret_cast<FwdWork*>(bwd_work);
    p.n_chunks = bwd_work + 4 * (size_t)L.max_chunks;
    p.first = bwd_work + L.off_first;
    p.len = bwd_work + L.off_len;
    p.groups = bwd_work + L.off_groups;
    p.rowinfo = reinterpret_cast<unsigned long long*>(bwd_work + L.off_rowinfo);
    p.lists = reinterpret_cast<unsigned short*>(bwd_work + L.off_lists);
    return p;
}

const int* ft_slice_outside_flag(int* fwd_work, int n_items, int N, int rps) {
    return slice_buffers(fwd_work, n_items, ceil_div(N, rps) + 1).outside_flag;
}

int launch_inverse_slice(cudaStream_t s, const int* item_seg, int* fwd_work, int* bwd_work, int B, int A, int N, int rps,
                         int n_persp) {
    if (B <= 0) return 0;
    const int n_items = n_persp * B;
    const int n_slices = ceil_div(N, rps), n_keys = n_slices + 1;
    const int A_pad = slice_a_pad(A);
    const SliceBuffers sb = slice_buffers(fwd_work, n_items, n_keys);
    const BwdLayout L = bwd_layout(n_items, A, rps);
    const BwdPointers P = bwd_pointers(bwd_work, L);
    k_chunk_plan<<<1, 128, 0, s>>>(item_seg, n_keys, L.CH, P.chunks, P.n_chunks, P.first, P.groups, L.max_groups);
    const int rps_h = (rps + 1) & ~1;
    const size_t inv_smem = (size_t)32 * rps_h * 2 + (size_t)INV_SORT_N * 4 * 2 + (size_t)L.region * 2;
    cudaFuncSetAttribute(k_inv_chunk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)inv_smem);
    k_inv_chunk<<<L.max_chunks, 1024, inv_smem, s>>>(reinterpret_cast<const unsigned short*>(sb.codes), P.chunks, P.n_chunks,
                                                     sb.outside_flag, n_slices, A_pad, rps, L.rps_pad, L.CH, L.region, P.lists,
                                                     P.rowinfo, P.len);
    return 2;
}

int launch_ft_backward_slice(cudaStream_t s, const void* dft_stm, const void* dft_nstm, int* fwd_work, int* bwd_work, int B,
                             int A, int N, int F, int rps, int n_persp, int slice_begin, int slice_count, float* grad, float* slabs,
                             int dft_half) {
    if (B <= 0) return 0;
    const int n_items = n_persp * B;
    const int n_slices = ceil_div(N, rps), n_keys = n_slices + 1;
    const int A_pad = slice_a_pad(A);
    const SliceBuffers sb = slice_buffers(fwd_work, n_items, n_keys);
    const BwdLayout L = bwd_layout(n_items, A, rps);
    const BwdPointers P = bwd_pointers(bwd_work, L);
    const size_t smem = bwd_smem_bytes(L.CH, rps, A_pad);
    if (slice_begin < 0 || slice_count <= 0 || slice_begin + slice_count > n_slices) return 0;
    const int grid_x = slice_count;  // a block row per slice; rows take the extra groups of shared slices in turn
    if (dft_half) {
        cudaFuncSetAttribute(k_ft_backward_slice<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k_ft_backward_slice<true><<<dim3(grid_x, F / 64), 1024, smem, s>>>(dft_stm, dft_nstm, sb.info, P.chunks, P.groups, P.len,
                                                                                 P.rowinfo, P.lists, sb.outside_flag, B, F, N, rps,
                                                                                 L.rps_pad, L.CH, L.region, slice_begin, slice_count, grad,
                                                                                 slabs);
    } else {
        cudaFuncSetAttribute(k_ft_backward_slice<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k_ft_backward_slice<false><<<dim3(grid_x, F / 32), 1024, smem, s>>>(dft_stm, dft_nstm, sb.info, P.chunks, P.groups, P.len,
                                                                                  P.rowinfo, P.lists, sb.outside_flag, B, F, N, rps,
                                                                                  L.rps_pad, L.CH, L.region, slice_begin, slice_count, grad,
                                                                                  slabs);
    }
    k_bwd_combine<<<dim3(148, slice_count), 256, 0, s>>>(P.groups, sb.outside_flag, reinterpret_cast<const float4*>(slabs),
                                                         reinterpret_cast<float4*>(grad), rps, F, N, slice_begin);
    return 2;
}
