// FT weight gradient for callers that are not allowed to allocate device memory.
//
// Some hosts of this library run inside a memory plan that is fixed before training starts: a framework
// whose caching allocator owns all of the GPU's memory, a process that shares the device with a
// latency-critical service and must not touch the driver's allocator on its hot path, or a harness that
// forbids cudaMalloc after start-up so that fragmentation cannot surprise it hours into a run.  Such a
// caller can hand over its own input and output buffers but has nowhere to get the working memory of the
// inverse index (histogram, offsets, cursors, position lists) from.
//
// tb_ft_backward_static_scratch therefore keeps that working memory in a file-scope __device__ array of a
// fixed size.  It calls no cudaMalloc / cudaFree and no allocating library routine.  The price:
//   - every GPU on which this library's device code is used holds the array (about 21.5 MB) from that first
//     use until the process exits;
//   - sizes are capped: ft_in <= TB_STATIC_SCRATCH_MAX_FT_IN rows, batch * max_active <=
//     TB_STATIC_SCRATCH_MAX_PAIRS index slots; larger problems are refused with an error text;
//   - all calls on one device share the one array, and it still holds whatever the previous call left
//     there.  The cells that must start at zero are cleared by every call, but two calls that overlap on
//     the GPU (different streams, or different host threads) race on it: serialise them.
//   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
//     first call outside of any stream capture.
#include "common.cuh"
#include "../../include/tatara_b200.h"

#include <stdio.h>

#include <mutex>

#define MAX_FT_IN TB_STATIC_SCRATCH_MAX_FT_IN
#define MAX_PAIRS TB_STATIC_SCRATCH_MAX_PAIRS
#define MAX_FT_OUT 4096
// layout expected by launch_inverse_index: histogram + long-list queue + scan sums, offsets [2(N + 1)],
// cursors [2N], lists + sort scratch [4P]; then what launch_ft_backward_split needs to cut long lists into parts:
// its plan [2 + 2 * max_work + 3N] and the partial rows [max_work][F]
#define COUNTS_INTS (4 * MAX_FT_IN + 1 + 2 * (MAX_FT_IN / 2048 + 2))
#define MAX_WORK (2 * (MAX_PAIRS / 4096) + 2)   /* ft_backward_max_work at the slot limit */
#define PLAN_INTS (2 + 2 * MAX_WORK + 3 * MAX_FT_IN)
#define SCRATCH_INTS (COUNTS_INTS + 4 * MAX_FT_IN + 2 + 4 * MAX_PAIRS + PLAN_INTS + MAX_WORK * MAX_FT_OUT + 64)

// In host code this name is only a handle for the runtime, not a device address: it must never be passed
// to a kernel.  The address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) int g_static_scratch[SCRATCH_INTS];

namespace {
std::mutex g_mu;
int* g_scratch_addr[64] = {nullptr};

int report(char* err, size_t err_len, int code, const char* fmt, long long a = 0, long long b = 0) {
    if (err && err_len) snprintf(err, err_len, fmt, a, b);
    return code;
}
}  // namespace

extern "C" int tb_ft_backward_static_scratch(const float* d_dft, const int32_t* d_indices, const int32_t* d_nnz,
                                             int batch, int ft_out, int ft_in, int max_active, float* d_grad,
                                             void* stream, char* err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (!d_dft || !d_indices || !d_nnz || !d_grad)
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT, "a device pointer is NULL");
    if (batch < 1 || max_active < 1 || ft_in < 1)
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT, "batch, max_active and ft_in must be positive");
    if (ft_out < 128 || ft_out % 128 != 0 || ft_out > MAX_FT_OUT)
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT, "ft_out must be a multiple of 128 in [128, 4096] (got %lld)", ft_out);
    if (((uintptr_t)d_dft | (uintptr_t)d_grad) & 15)
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT, "d_dft and d_grad must be 16-byte aligned (rows are moved as 128-bit vectors)");
    if (ft_in > MAX_FT_IN)
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT,
                      "ft_in %lld exceeds the static scratch limit of %lld rows (use the allocating entry points)", ft_in, MAX_FT_IN);
    if ((long long)batch * max_active > MAX_PAIRS)
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT,
                      "batch * max_active = %lld exceeds the static scratch limit of %lld index slots", (long long)batch * max_active,
                      MAX_PAIRS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return report(err, err_len, TB_ERR_NO_DEVICE, "no current CUDA device");
    int* base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_addr[dev]) {
            // once per device, with that device current: the array's address in THIS device's memory
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess) {
                if (err && err_len) snprintf(err, err_len, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
                return TB_ERR_CUDA;
            }
            g_scratch_addr[dev] = static_cast<int*>(p);
        }
        base = g_scratch_addr[dev];
    }
    const size_t N = (size_t)ft_in, P = (size_t)batch * max_active;
    int* counts = base;                                         // [inverse_index_counts_len(N)]
    int* offsets = counts + inverse_index_counts_len(ft_in);    // [2(N + 1)]
    int* cursor = offsets + 2 * (N + 1);      // [2N]
    int* lists = cursor + 2 * N;              // [4P]
    // The plan holds 8-byte records and the partial rows are moved as float4: both start on a 16-byte boundary of the
    // array itself (offsets from its 256-byte aligned base rounded up to a multiple of four ints).
    const size_t max_work = (size_t)ft_backward_max_work(batch, max_active, 1);  // <= MAX_WORK by the slot limit
    const size_t plan_off = ((size_t)(lists - base) + 4 * P + 3) / 4 * 4;
    const size_t partial_off = (plan_off + 2 + 2 * max_work + 3 * N + 3) / 4 * 4;
    int* plan = base + plan_off;              // [2 + 2 * max_work + 3N]
    float* partial = reinterpret_cast<float*>(base + partial_off);
    if (partial_off + max_work * (size_t)ft_out > (size_t)SCRATCH_INTS)   // cannot happen inside the limits checked above
        return report(err, err_len, TB_ERR_INVALID_ARGUMENT, "static scratch layout overflow");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // launch_inverse_index clears the histogram and the long-list counter itself, launch_ft_backward_split its two
    // counters; offsets, cursors, lists, plan and partial rows are rewritten for the rows and slots this call uses
    launch_inverse_index(s, nullptr, d_indices, d_indices, d_nnz, batch, max_active, ft_in, 1, counts, offsets, cursor, lists);
    // the same launcher as tb_ft_backward_bench: lists of more than 4096 entries are summed in parts of 4096
    launch_ft_backward_split(s, nullptr, d_dft, d_dft, offsets, lists, batch, max_active, ft_in, ft_out, 1, plan, partial, d_grad);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        if (err && err_len) snprintf(err, err_len, "kernel launch: %s", cudaGetErrorString(e));
        return TB_ERR_CUDA;
    }
    return TB_OK;
}
