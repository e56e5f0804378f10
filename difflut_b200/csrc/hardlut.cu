// Bit-packed hard-LUT inference helpers: class counts from packed layer outputs.
//
// The reference has no packed path; its eval mode produces fp32 {0,1} node outputs and sums them
// with GroupSum (difflut/nodes/dwn_node.py:457-483, difflut/utils/modules.py:116-163).  Here the
// last layer's packed output bits [N][Bp/32] are counted per class into int32.
#include "common.cuh"

namespace {

// thread per (class, sample): lanes of a warp share the word they read, so each row costs one
// broadcast load per 32 samples.
__global__ void popcount_groupsum_kernel(const uint32_t* __restrict__ bits_t, int32_t* __restrict__ counts,
                                         int64_t N, int k, int64_t gsz, int64_t B, int64_t Wp) {
    const int64_t total = (int64_t)k * (Wp * 32);
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = t / (Wp * 32), b = t - c * (Wp * 32);
        if (b >= B) continue;
        int64_t r1 = (c + 1) * gsz;
        if (r1 > N) r1 = N;
        const int64_t w = b >> 5;
        const int sh = (int)(b & 31);
        int cnt = 0;
        for (int64_t r = c * gsz; r < r1; ++r) cnt += (__ldg(bits_t + r * Wp + w) >> sh) & 1u;
        counts[b * k + c] = cnt;
    }
}

}  // namespace

DL_EXPORT int dl_popcount_groupsum_t(const uint32_t* bits_t, int32_t* counts, int64_t N, int64_t k,
                                     int64_t B, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(bits_t && counts && N > 0 && k > 0 && B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    const int64_t gsz = dl_ceil_div(N, k);
    const int64_t blocks = dl_min64(dl_ceil_div(k * Bp, 256), (int64_t)DL_NUM_SMS * 32);
    popcount_groupsum_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(bits_t, counts, N, (int)k, gsz, B,
                                                                          Bp / 32);
    return dl_launch_status();
}
