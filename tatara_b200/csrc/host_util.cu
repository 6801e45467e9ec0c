// Host-side helpers of the C ABI that need no GPU: the reference's deterministic weight initialiser.
#include "../../include/tatara_b200.h"

#include <math.h>
#include <string.h>

// crates/nnue-train/src/init.rs:111-210: xorshift64 (13, 7, 17), top 53 bits as an f32 unit value,
// uniform in [-h, +h]; `per_bucket_repeat` samples one bucket and tiles it over all buckets.
// dist: 0 zeroed, 1 uniform.  scale_kind: 0 absolute half width, 1 sqrt(gain / fan_in).
extern "C" int tb_init_sample(float* out, int64_t n, int64_t num_buckets, int64_t fan_in, int dist, int scale_kind,
                              float scale_value, int per_bucket_repeat, uint64_t seed) {
    if (n < 0 || (n > 0 && !out)) return TB_ERR_INVALID_ARGUMENT;
    if (dist == 0) { memset(out, 0, (size_t)n * sizeof(float)); return TB_OK; }
    if (dist != 1) return TB_ERR_UNSUPPORTED;
    float mag = scale_value;
    if (scale_kind == 1) mag = sqrtf(scale_value / (float)(fan_in < 1 ? 1 : fan_in));
    int64_t block = n;
    if (per_bucket_repeat) {
        if (num_buckets < 1 || n % num_buckets != 0) return TB_ERR_INVALID_ARGUMENT;
        block = n / num_buckets;
    }
    uint64_t s = seed < 1 ? 1 : seed;
    for (int64_t i = 0; i < block; ++i) {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        const float u = (float)(s >> 11) / (float)(1ull << 53);
        out[i] = (u * 2.0f - 1.0f) * mag;
    }
    if (per_bucket_repeat)
        for (int64_t g = 1; g < num_buckets; ++g) memcpy(out + g * block, out, (size_t)block * sizeof(float));
    return TB_OK;
}
