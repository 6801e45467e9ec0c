// L1 forward on the 5th-generation tensor cores (tcgen05, TF32 operands, fp32 accumulators in tensor memory), used
// when the trainer runs with --tf32 (bins/nnue_train/src/cli.rs:623-638; the reference then runs its L1 products as
// cuBLAS Sgemm calls in TF32 tensor-op mode, one per bucket segment plus one for the shared layer:
// bins/nnue_train/src/trainer_layerstack.rs:2388-2420, 2498-2506, bins/nnue_train/src/trainer_common.rs:691-727).
//
// Same contraction as k_l1_forward_stream: y[pos, :] = beff[g] + x[pos, :] . weff[g]^T with the effective weights
// weff[g] = wb[g] + ws^T of the position's bucket g.  A block owns 128 consecutive positions of the bucket order (one
// bucket), i.e. one 128 x l1 accumulator tile in tensor memory; x rows are reached through `order`, so the operands are
// staged by 16-byte asynchronous copies straight into the tensor cores' canonical K-major layout without swizzle: core
// matrices of 8 rows x 16 bytes, stored contiguously; the next 16 bytes along K lie 128 bytes further (leading byte
// offset), the next 8 rows TC_KC / 4 core matrices further (stride byte offset).  One thread issues the MMAs of a K chunk
// (M = 128, N = l1 or 16, K = 8 each) and commits them to the stage's mbarrier, which frees the stage for the copies of
// a later chunk.  TF32 operands are the fp32 values as they are: the tensor cores read the upper 19 bits.
// The contraction is read-bound (l1 <= 32 output columns): the tensor pipe is nearly idle by construction; what the
// tensor cores buy is an instruction stream of copies only, so that the x rows stream at HBM speed.
//
// Every wait on an mbarrier is bounded; a wait that runs out raises *error_flag and the block carries on to its normal
// exit (all further waits are bounded too), where tensor memory is released.
#include "common.cuh"

#define TC_POS 128   // positions per block = rows of the accumulator tile
#define TC_KC 32     // fp32 elements per stage along K: four MMAs of K = 8
#define TC_STAGES 3
#define TC_WAIT_LIMIT (1 << 18)

namespace {

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_cp16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// bounded wait for the completion of the phase with the given parity; false when the limit ran out
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (int i = 0; i < TC_WAIT_LIMIT; ++i) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// shared-memory matrix descriptor: K-major, no swizzle, start address / leading / stride byte offsets in 16-byte units,
// descriptor version 1 (bits 46-47)
__device__ __forceinline__ unsigned long long umma_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    return (unsigned long long)((addr & 0x3FFFFu) >> 4) | ((unsigned long long)(lbo_bytes >> 4) << 16) |
           ((unsigned long long)(sbo_bytes >> 4) << 32) | (1ull << 46);
}

}  // namespace

template <int L1>
__global__ void __launch_bounds__(128) k_l1_forward_tc(const float* __restrict__ x, int K, const int* __restrict__ order,
                                                        const TileDesc* __restrict__ tiles, const TileDesc* __restrict__ units,
                                                        const int* __restrict__ n_units, const float* __restrict__ weff,
                                                        const float* __restrict__ beff, float* __restrict__ y, int nb,
                                                        int* __restrict__ error_flag) {
    constexpr int NB = L1 < 16 ? 16 : L1;             // N of the MMA (a multiple of 16 for M = 128)
    constexpr int A_BYTES = TC_POS * TC_KC * 4;       // 16 KB
    constexpr int B_BYTES = NB * TC_KC * 4;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned LBO = 128, SBO = (TC_KC / 4) * 128;
    // instruction descriptor: fp32 accumulator (bits 4-5 = 1), TF32 A and B (bits 7-9, 10-12 = 2), both K-major,
    // N >> 3 at bit 17, M >> 4 at bit 24
    constexpr unsigned IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(NB >> 3) << 17) | ((unsigned)(TC_POS >> 4) << 24);
    extern __shared__ __align__(16) unsigned char s_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[TC_STAGES];
    __shared__ unsigned s_tmem;
    __shared__ int s_pos[TC_POS];

    const int u = blockIdx.x >> 1, h = blockIdx.x & 1;
    if (u >= *n_units) return;
    const TileDesc ud = units[u];
    const int per = TC_POS / TB_TILE_M;
    const int first = ud.start + h * per, last = min(ud.start + ud.count, first + per);
    if (first >= last) return;
    const int p_begin = tiles[first].start;
    const int n = tiles[last - 1].start + tiles[last - 1].count - p_begin;
    const int g = ud.bucket < nb ? ud.bucket : nb;
    const int tid = threadIdx.x, warp = tid >> 5;
    const unsigned ring = (smem_u32(s_dyn) + 127u) & ~127u;  // stage buffers on a 128-byte boundary

    for (int i = tid; i < TC_POS; i += 128) s_pos[i] = order[p_begin + (i < n ? i : 0)];  // rows past the end repeat the first
    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_bar[s])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {  // tensor memory: 32 columns (the smallest allocation) hold the 128 x NB fp32 tile
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if constexpr (L1 < NB) {  // weight rows l1 .. 15 of every stage stay zero
        constexpr int PAD = NB - L1;
        for (int e = tid; e < TC_STAGES * PAD * (TC_KC / 4); e += 128) {
            const int s = e / (PAD * (TC_KC / 4)), r = L1 + (e / (TC_KC / 4)) % PAD, kc = e % (TC_KC / 4);
            unsigned char* p = s_dyn + (ring - smem_u32(s_dyn)) + (size_t)s * STAGE_BYTES + A_BYTES + (r >> 3) * SBO + kc * LBO + (r & 7) * 16;
            *reinterpret_cast<float4*>(p) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = s_tmem;

    // this thread's copies of one chunk: the 16-byte piece kc of rows r0 + 16 i (i < 8) of x, and of the weight rows
    const int kc = tid & 7, r0 = tid >> 3;
    const float* __restrict__ wg = weff + (size_t)g * L1 * K;
    const float* xrow[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) xrow[i] = x + (size_t)s_pos[r0 + 16 * i] * K + 4 * kc;
    const int nk = K / TC_KC;
    bool failed = false;
    auto issue = [&](int c) {
        if (c < nk) {
            const int s = c % TC_STAGES;
            // the stage's previous chunk (c - TC_STAGES) must have been consumed by its MMAs
            // (after one wait has run out no other is started: the block only drains)
            if (c >= TC_STAGES && !failed && !mbar_wait(smem_u32(&s_bar[s]), (unsigned)((c / TC_STAGES - 1) & 1))) failed = true;
            const unsigned a_base = ring + s * STAGE_BYTES, b_base = a_base + A_BYTES;
            const int k0 = c * TC_KC;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = r0 + 16 * i;
                tc_cp16(a_base + (r >> 3) * SBO + kc * LBO + (r & 7) * 16, xrow[i] + k0);
            }
            for (int r = r0; r < L1; r += 16) tc_cp16(b_base + (r >> 3) * SBO + kc * LBO + (r & 7) * 16, wg + (size_t)r * K + k0 + 4 * kc);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // one group per chunk, empty past the end
    };
#pragma unroll
    for (int c = 0; c < TC_STAGES - 1; ++c) issue(c);
    for (int c = 0; c < nk; ++c) {
        issue(c + TC_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(TC_STAGES - 1) : "memory");  // this thread's copies of chunk c have landed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");              // ... and are visible to the tensor cores
        __syncthreads();                                                           // every thread's copies of chunk c
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int s = c % TC_STAGES;
            const unsigned a_base = ring + s * STAGE_BYTES, b_base = a_base + A_BYTES;
#pragma unroll
            for (int j = 0; j < TC_KC / 8; ++j) {
                const unsigned long long da = umma_desc(a_base + j * 2 * LBO, LBO, SBO), db = umma_desc(b_base + j * 2 * LBO, LBO, SBO);
                const unsigned acc = (c > 0 || j > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                    ::"r"(tmem), "l"(da), "l"(db), "r"(IDESC), "r"(acc)
                    : "memory");
            }
            // arrives on the stage's barrier when these (and all earlier) MMAs are done with the stage's memory
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s_bar[s])) : "memory");
        }
        __syncwarp();  // the issuing thread's warp mates wait for it here, not in a spin on the barrier it is about to signal
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the last chunk's commit covers every MMA of the block
    if (!failed && !mbar_wait(smem_u32(&s_bar[(nk - 1) % TC_STAGES]), (unsigned)(((nk - 1) / TC_STAGES) & 1))) failed = true;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (failed) atomicExch(error_flag, 1);
    __syncwarp();  // the tensor-memory loads below want the whole warp

    // epilogue: warp w reads lanes 32 w .. 32 w + 31 of the tile, a lane = a position, 16 columns per load
    const int row = tid;
    const unsigned taddr = tmem + ((unsigned)(warp * 32) << 16);
#pragma unroll
    for (int c0 = 0; c0 < L1; c0 += 16) {
        unsigned v[16];
        __syncwarp();
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
              "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr + (unsigned)c0));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < n) {
            float* yr = y + (size_t)s_pos[row] * L1 + c0;
            const float* bg = beff + (size_t)g * L1 + c0;
            constexpr int NC = L1 - 0 < 16 ? L1 : 16;  // columns of this load that exist (l1 = 8: the first eight)
#pragma unroll
            for (int o = 0; o < NC; o += 4)
                *reinterpret_cast<float4*>(yr + o) = make_float4(__uint_as_float(v[o]) + bg[o], __uint_as_float(v[o + 1]) + bg[o + 1],
                                                                 __uint_as_float(v[o + 2]) + bg[o + 2], __uint_as_float(v[o + 3]) + bg[o + 3]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
}

bool l1_forward_tc_supported(int K, int l1) { return (l1 == 8 || l1 == 16 || l1 == 32) && K % TC_KC == 0 && K / TC_KC >= TC_STAGES; }

// weff / beff: the effective weights and biases k_l1_weff has built for this step
int launch_l1_forward_tc(cudaStream_t s, const float* x, int K, const int* order, const TileDesc* tiles, const int* n_tiles,
                         int max_tiles, const float* weff, const float* beff, float* y, int l1, int nb, int* error_flag) {
    const int max_units = sort_max_units(max_tiles);
    const TileDesc* units = tiles + max_tiles;
    const int NB = l1 < 16 ? 16 : l1;
    const size_t smem = (size_t)TC_STAGES * (TC_POS + NB) * TC_KC * 4 + 128;
#define TC_LAUNCH(L)                                                                                                    \
    do {                                                                                                                \
        cudaFuncSetAttribute(k_l1_forward_tc<L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
        k_l1_forward_tc<L><<<2 * max_units, 128, smem, s>>>(x, K, order, tiles, units, n_tiles + 1, weff, beff, y, nb, error_flag); \
    } while (0)
    if (l1 == 8) TC_LAUNCH(8); else if (l1 == 16) TC_LAUNCH(16); else TC_LAUNCH(32);
#undef TC_LAUNCH
    return 1;
}
