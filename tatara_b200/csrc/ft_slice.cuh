// Shared pieces of the slice-resident FT kernels (forward in ft_kernels.cu, weight gradient in ft_slice_bwd.cu).
#pragma once
#include "common.cuh"

#define SLICE_IPC 4096           // items per block of the forward (a multiple of 128): at 65 536 positions a slice of the
                                 // benchmark (2 900 items) is one run, its strip is loaded once (2048: two runs, 0.03 ms slower)
#define SORT_KEYS_LIMIT 128      // key limit of the small-key sorts (sort_kernels.cu): slices + 1
#define SLICE_OUTSIDE 0xFFFFu    // row code: the feature's table row lies outside the item's slice
#define SLICE_SLOW_BIT 0x40000000  // info[slot] bit: the item has such a row

// a run of consecutive slots of the sorted item list that belong to one slice
struct FwdWork {
    int slice, begin, end, pad;
};

static inline int slice_a_pad(int A) { return (A + 7) / 8 * 8; }
static inline size_t slice_max_work(int n_items, int n_keys) { return (size_t)n_items / SLICE_IPC + n_keys + 2; }

// layout of the forward's work buffer (ft_forward_slice_work_ints): the weight-gradient kernels read info and codes
struct SliceBuffers {
    FwdWork* work;
    int* n_work;        // [0] number of records
    int* outside_flag;  // 1 when some item has a row outside its slice
    int* info;          // [n_items] item of every slot (| SLICE_SLOW_BIT)
    uint4* codes;       // [n_items][A_pad] 16-bit row codes
};
static inline SliceBuffers slice_buffers(int* work, int n_items, int n_keys) {
    SliceBuffers b;
    const size_t max_work = slice_max_work(n_items, n_keys);
    b.work = reinterpret_cast<FwdWork*>(work);
    b.n_work = work + 4 * max_work;
    b.outside_flag = b.n_work + 1;
    b.info = b.n_work + 4;                                                             // 16-byte aligned
    b.codes = reinterpret_cast<uint4*>(b.info + ((size_t)n_items + 3) / 4 * 4);        // 16-byte aligned
    return b;
}

#ifdef __CUDACC__
#include <cuda_fp16.h>
// two fp32 additions in one instruction (sm_100 packed arithmetic); each half is an IEEE round-to-nearest add
static __device__ __forceinline__ unsigned long long fadd2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
static __device__ __forceinline__ float lo_f(unsigned long long v) { return __uint_as_float((unsigned)v); }
static __device__ __forceinline__ float hi_f(unsigned long long v) { return __uint_as_float((unsigned)(v >> 32)); }
// acc += (float)h for the two fp16 values packed in `pair`: sm_100's mixed-precision add takes the fp16 operand as it is
// (the conversion is exact, so each is the IEEE fp32 add of the converted value)
static __device__ __forceinline__ void add_h2(float& a_lo, float& a_hi, unsigned pair) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tadd.rn.f32.f16 %0, l, %0;\n\tadd.rn.f32.f16 %1, h, %1;\n\t}"
        : "+f"(a_lo), "+f"(a_hi)
        : "r"(pair));
}
static __device__ __forceinline__ unsigned pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&h);
}
static __device__ __forceinline__ float2 unpack_h2(unsigned pair) { return __half22float2(*reinterpret_cast<const __half2*>(&pair)); }

// The running sums of one lane of the slice-resident FT kernels.  A lane reads 16 bytes of every row from shared memory:
// four fp32 columns (two packed f32x2 accumulators) or eight fp16 columns (eight fp32 accumulators; fp16 rows are summed
// in fp32, native_kernels.cu:743-801, :1081-1140).
template <bool HALF>
struct LaneAcc;
template <>
struct LaneAcc<false> {
    static constexpr int COLS = 4;
    unsigned long long a0, a1;
    __device__ __forceinline__ void zero() { a0 = 0ull; a1 = 0ull; }
    __device__ __forceinline__ void add(const ulonglong2& v) { a0 = fadd2(a0, v.x); a1 = fadd2(a1, v.y); }
    __device__ __forceinline__ void add(const LaneAcc& o) { a0 = fadd2(a0, o.a0); a1 = fadd2(a1, o.a1); }
    __device__ __forceinline__ void add_from(const LaneAcc& base) { a0 = fadd2(base.a0, a0); a1 = fadd2(base.a1, a1); }  // this = base + this
    __device__ __forceinline__ LaneAcc shfl_xor(int m) const {
        LaneAcc r;
        r.a0 = __shfl_xor_sync(0xffffffffu, a0, m);
        r.a1 = __shfl_xor_sync(0xffffffffu, a1, m);
        return r;
    }
    __device__ __forceinline__ float get(int i) const { return i == 0 ? lo_f(a0) : i == 1 ? hi_f(a0) : i == 2 ? lo_f(a1) : hi_f(a1); }
    // running sums live in fp32 gradient rows
    __device__ __forceinline__ void load_cg(const float* p) {
        const ulonglong2 v = __ldcg(reinterpret_cast<const ulonglong2*>(p));
        a0 = v.x; a1 = v.y;
    }
    __device__ __forceinline__ void store_cg(float* p) const { __stcg(reinterpret_cast<ulonglong2*>(p), make_ulonglong2(a0, a1)); }
};
template <>
struct LaneAcc<true> {
    static constexpr int COLS = 8;
    float a[8];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.f;
    }
    __device__ __forceinline__ void add(const ulonglong2& v) {
        add_h2(a[0], a[1], (unsigned)v.x); add_h2(a[2], a[3], (unsigned)(v.x >> 32));
        add_h2(a[4], a[5], (unsigned)v.y); add_h2(a[6], a[7], (unsigned)(v.y >> 32));
    }
    __device__ __forceinline__ void add(const LaneAcc& o) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += o.a[i];
    }
    __device__ __forceinline__ void add_from(const LaneAcc& base) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = base.a[i] + a[i];
    }
    __device__ __forceinline__ LaneAcc shfl_xor(int m) const {
        LaneAcc r;
#pragma unroll
        for (int i = 0; i < 8; ++i) r.a[i] = __shfl_xor_sync(0xffffffffu, a[i], m);
        return r;
    }
    __device__ __forceinline__ float get(int i) const { return a[i]; }
    __device__ __forceinline__ void load_cg(const float* p) {
        const float4 u = __ldcg(reinterpret_cast<const float4*>(p)), w = __ldcg(reinterpret_cast<const float4*>(p) + 1);
        a[0] = u.x; a[1] = u.y; a[2] = u.z; a[3] = u.w; a[4] = w.x; a[5] = w.y; a[6] = w.z; a[7] = w.w;
    }
    __device__ __forceinline__ void store_cg(float* p) const {
        __stcg(reinterpret_cast<float4*>(p), make_float4(a[0], a[1], a[2], a[3]));
        __stcg(reinterpret_cast<float4*>(p) + 1, make_float4(a[4], a[5], a[6], a[7]));
    }
};

// asynchronous 16-byte copy global -> shared; src_bytes = 0 writes zeros and reads nothing
static __device__ __forceinline__ void cp_async16(void* dst_shared, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((unsigned)__cvta_generic_to_shared(dst_shared)), "l"(src),
                 "r"(src_bytes)
                 : "memory");
}
static __device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_PENDING>
static __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_PENDING) : "memory"); }
#endif
