// Shared pieces of the slice-resident FT kernels (forward in ft_kernels.cu, weight gradient in ft_slice_bwd.cu).
#pragma once
#include "common.cuh"

#define SLICE_IPC 2048           // items per block of the forward (a multiple of 128)
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
// two fp32 additions in one instruction (sm_100 packed arithmetic); each half is an IEEE round-to-nearest add
static __device__ __forceinline__ unsigned long long fadd2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
static __device__ __forceinline__ float lo_f(unsigned long long v) { return __uint_as_float((unsigned)v); }
static __device__ __forceinline__ float hi_f(unsigned long long v) { return __uint_as_float((unsigned)(v >> 32)); }
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
