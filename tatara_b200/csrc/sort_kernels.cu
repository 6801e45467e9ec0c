// Small-key stable counting sorts over many blocks (keys < 128):
//  - positions by LayerStack bucket  -> `order`, bucket segments, dense tiles and work units
//    (replaces count_buckets / exclusive_scan_aligned / scatter_bucket_perm, native_kernels.cu:1858-1925)
//  - (position, perspective) items by the king bucket of their feature rows -> `items`, so that blocks that
//    run at the same time gather from the same slice of the FT table and the slice stays in L2.
// Both sorts share three launches (blockIdx.y / blockIdx.x selects the sort): per-block histogram, one-block scan of the
// [key][block] matrix, stable scatter (rank inside a block = warp match + prefix over the block's warps); a fourth
// launch cuts the bucket segments into tiles and work units.  Results do not depend on timing.
#include "common.cuh"

#define SORT_BLOCK 1024
#define SORT_MAX_KEYS 128

struct BucketKey {
    const int* bucket;  // may be NULL: one group
    int nb;
    __device__ int operator()(int i) const {
        const int k = bucket ? bucket[i] : 0;
        return (unsigned)k < (unsigned)nb ? k : nb;  // out-of-range ids form the last group
    }
};

// item i < B is the stm perspective of position i, item B + b the nstm perspective of position b.  The key is
// the table slice (index / rows_per_slice) of the item's first feature; items without one go last.
struct ItemKey {
    const int* idx_stm;
    const int* idx_nstm;
    const int* nnz;
    int B, A, N, rows_per_slice, n_slices;
    __device__ int operator()(int i) const {
        const int p = i >= B, b = i - p * B;
        if (nnz[b] <= 0) return n_slices;
        const int f = (p ? idx_nstm : idx_stm)[(size_t)b * A];
        return (unsigned)f < (unsigned)N ? f / rows_per_slice : n_slices;
    }
};

template <class KeyFn>
static __device__ __forceinline__ void sort_hist_body(KeyFn fn, int n, int K, int G, int* __restrict__ hist, int* s_h, int block) {
    if (threadIdx.x < SORT_MAX_KEYS) s_h[threadIdx.x] = 0;
    __syncthreads();
    const int i = block * SORT_BLOCK + threadIdx.x;
    if (i < n) atomicAdd(&s_h[fn(i)], 1);
    __syncthreads();
    if ((int)threadIdx.x < K) hist[threadIdx.x * G + block] = s_h[threadIdx.x];
}

// two independent sorts in one launch: blockIdx.y selects the sort
template <class Fn0, class Fn1>
__global__ void __launch_bounds__(SORT_BLOCK) k_sort_hist2(Fn0 f0, int n0, int K0, int G0, int* __restrict__ h0, Fn1 f1, int n1, int K1,
                                                            int G1, int* __restrict__ h1) {
    __shared__ int s_h[SORT_MAX_KEYS];
    if (blockIdx.y == 0) { if ((int)blockIdx.x < G0) sort_hist_body(f0, n0, K0, G0, h0, s_h, blockIdx.x); }
    else if ((int)blockIdx.x < G1) sort_hist_body(f1, n1, K1, G1, h1, s_h, blockIdx.x);
}

// exclusive scan of hist[K][G] in key-major order (in place); seg_start[k] = first output slot of key k
static __device__ __forceinline__ void sort_scan_body(int* __restrict__ hist, int K, int G, int n, int* __restrict__ seg_start, int* s_warp) {
    const int total = K * G;
    const int per = (total + 1023) / 1024;
    const int beg = min((int)threadIdx.x * per, total), end = min(beg + per, total);
    int sum = 0;
    for (int i = beg; i < end; ++i) sum += hist[i];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int incl = sum;
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
    int run = s_warp[w] + incl - sum;
    for (int i = beg; i < end; ++i) {
        const int c = hist[i];
        hist[i] = run;
        if (i % G == 0) seg_start[i / G] = run;
        run += c;
    }
    if (threadIdx.x == 0) seg_start[K] = n;
}

__global__ void __launch_bounds__(1024) k_sort_scan2(int* __restrict__ h0, int K0, int G0, int n0, int* __restrict__ seg0,
                                                      int* __restrict__ h1, int K1, int G1, int n1, int* __restrict__ seg1) {
    __shared__ int s_warp[32];
    if (blockIdx.x == 0) sort_scan_body(h0, K0, G0, n0, seg0, s_warp);
    else sort_scan_body(h1, K1, G1, n1, seg1, s_warp);
}

template <class KeyFn>
static __device__ __forceinline__ void sort_scatter_body(KeyFn fn, int n, int K, int G, const int* __restrict__ base, int* __restrict__ out,
                                                         int (*s_cnt)[SORT_MAX_KEYS], int block) {
    for (int e = threadIdx.x; e < 32 * SORT_MAX_KEYS; e += SORT_BLOCK) (&s_cnt[0][0])[e] = 0;
    __syncthreads();
    const int i = block * SORT_BLOCK + threadIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int key = i < n ? fn(i) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (rank == 0 && key >= 0) s_cnt[w][key] = __popc(peers);
    __syncthreads();
    if ((int)threadIdx.x < K) {
        int run = 0;
        for (int ww = 0; ww < 32; ++ww) {
            const int c = s_cnt[ww][threadIdx.x];
            s_cnt[ww][threadIdx.x] = run;
            run += c;
        }
    }
    __syncthreads();
    if (key >= 0) out[base[key * G + block] + s_cnt[w][key] + rank] = i;
}

template <class Fn0, class Fn1>
__global__ void __launch_bounds__(SORT_BLOCK) k_sort_scatter2(Fn0 f0, int n0, int K0, int G0, const int* __restrict__ b0, int* __restrict__ o0,
                                                              Fn1 f1, int n1, int K1, int G1, const int* __restrict__ b1, int* __restrict__ o1) {
    __shared__ int s_cnt[32][SORT_MAX_KEYS];
    if (blockIdx.y == 0) { if ((int)blockIdx.x < G0) sort_scatter_body(f0, n0, K0, G0, b0, o0, s_cnt, blockIdx.x); }
    else if ((int)blockIdx.x < G1) sort_scatter_body(f1, n1, K1, G1, b1, o1, s_cnt, blockIdx.x);
}

// tiles: runs of <= TB_TILE_M positions of one bucket; units: runs of <= TB_UNIT_TILES tiles of one bucket
__global__ void __launch_bounds__(256) k_make_tiles(const int* __restrict__ seg_start, int K, TileDesc* __restrict__ tiles,
                                                     int* __restrict__ n_tiles, TileDesc* __restrict__ units,
                                                     int* __restrict__ n_units) {
    __shared__ int s_tile_base[SORT_MAX_KEYS + 1], s_unit_base[SORT_MAX_KEYS + 1], s_seg[SORT_MAX_KEYS + 2];
    for (int k = threadIdx.x; k <= K; k += blockDim.x) s_seg[k] = seg_start[k];  // one round trip, not K
    __syncthreads();
    if (threadIdx.x == 0) {
        int trun = 0, urun = 0;
        for (int k = 0; k < K; ++k) {
            s_tile_base[k] = trun;
            s_unit_base[k] = urun;
            const int nt = (s_seg[k + 1] - s_seg[k] + TB_TILE_M - 1) / TB_TILE_M;
            trun += nt;
            urun += (nt + TB_UNIT_TILES - 1) / TB_UNIT_TILES;
        }
        *n_tiles = trun;
        *n_units = urun;
    }
    __syncthreads();
    for (int k = 0; k < K; ++k) {
        const int s0 = s_seg[k], c = s_seg[k + 1] - s0;
        const int nt = (c + TB_TILE_M - 1) / TB_TILE_M;
        for (int t = threadIdx.x; t < nt; t += blockDim.x) {
            TileDesc d;
            d.start = s0 + t * TB_TILE_M;
            d.count = min(TB_TILE_M, c - t * TB_TILE_M);
            d.bucket = k;
            d.pad = 0;
            tiles[s_tile_base[k] + t] = d;
        }
        const int nu = (nt + TB_UNIT_TILES - 1) / TB_UNIT_TILES;
        for (int u = threadIdx.x; u < nu; u += blockDim.x) {
            TileDesc d;
            d.start = s_tile_base[k] + u * TB_UNIT_TILES;
            d.count = min(TB_UNIT_TILES, nt - u * TB_UNIT_TILES);
            d.bucket = k;
            d.pad = 0;
            units[s_unit_base[k] + u] = d;
        }
    }
}

int sort_max_units(int max_tiles) { return max_tiles / TB_UNIT_TILES + TB_MAX_BUCKETS + 2; }

// Both sorts of a step in four launches: positions by bucket (order, tiles, units) and items by table slice.
// hist: scratch of (nb + 1) * ceil(B / 1024) + (slices + 1) * ceil(n_persp * B / 1024) ints.
int launch_step_sorts(cudaStream_t s, const int* bucket, int B, int nb, int* order, TileDesc* tiles, int* n_tiles, int* seg_start,
                      int max_tiles, const int* idx_stm, const int* idx_nstm, const int* nnz, int A, int N, int rows_per_slice,
                      int n_persp, int* items, int* item_seg, int* hist) {
    int n_slices = ceil_div(N, rows_per_slice);
    if (n_slices + 1 > SORT_MAX_KEYS) {
        rows_per_slice = ceil_div(N, SORT_MAX_KEYS - 1);
        n_slices = ceil_div(N, rows_per_slice);
    }
    const int K0 = nb + 1, G0 = ceil_div(B, SORT_BLOCK);
    const int n1 = n_persp * B, K1 = n_slices + 1, G1 = ceil_div(n1, SORT_BLOCK);
    int* h0 = hist;
    int* h1 = hist + (size_t)K0 * G0;
    BucketKey f0{bucket, nb};
    ItemKey f1{idx_stm, idx_nstm, nnz, B, A, N, rows_per_slice, n_slices};
    const dim3 grid(G0 > G1 ? G0 : G1, 2);
    k_sort_hist2<<<grid, SORT_BLOCK, 0, s>>>(f0, B, K0, G0, h0, f1, n1, K1, G1, h1);
    k_sort_scan2<<<2, 1024, 0, s>>>(h0, K0, G0, B, seg_start, h1, K1, G1, n1, item_seg);
    k_sort_scatter2<<<grid, SORT_BLOCK, 0, s>>>(f0, B, K0, G0, h0, order, f1, n1, K1, G1, h1, items);
    k_make_tiles<<<1, 256, 0, s>>>(seg_start, K0, tiles, n_tiles, tiles + max_tiles, n_tiles + 1);
    return 4;
}
