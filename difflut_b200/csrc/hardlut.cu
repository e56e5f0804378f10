// Bit-packed hard-LUT inference helpers: class counts from packed layer outputs.
//
// The reference has no packed path; its eval mode produces fp32 {0,1} node outputs and sums them
// with GroupSum (difflut/nodes/dwn_node.py:457-483, difflut/utils/modules.py:116-163).  Here the
// last layer's packed output bits [N][Bp/32] are counted per class into int32.
#include "common.cuh"

namespace {

// full adder on 32 bit-columns at once: (h, l) = a + b + c
__device__ __forceinline__ void csa(uint32_t& h, uint32_t& l, uint32_t a, uint32_t b, uint32_t c) {
    const uint32_t u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}

// Eight threads per (class, word of 32 samples).  The class's rows are added bit-sliced: 16 rows at a time
// go through a carry-save adder tree into the planes ones / twos / fours / eights, the resulting
// sixteens word is rippled into six higher planes; at the end the planes are read out per sample.
// About 3 logic ops per row and word instead of 3 per row and SAMPLE.
__global__ void __launch_bounds__(128)
popcount_groupsum_kernel(const uint32_t* __restrict__ bits_t, int32_t* __restrict__ counts, int64_t N, int k,
                         int64_t gsz, int64_t B, int64_t Wp) {
    // 8 threads (consecutive lanes) share one (class, word): each takes every 8th block of 16 rows
    const int64_t total = (int64_t)k * Wp * 8;
    for (int64_t t8 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t8 < ((total + 31) & ~(int64_t)31);
         t8 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = t8 >> 3;
        const int part = (int)(t8 & 7);
        const bool live = t8 < total;
        const int64_t c = live ? t / Wp : 0, w = live ? t - c * Wp : 0;
        int64_t r1 = (c + 1) * gsz;
        if (r1 > N) r1 = N;
        if (!live || w * 32 >= B) r1 = 0;
        uint32_t ones = 0, twos = 0, fours = 0, eights = 0, hi[6] = {0, 0, 0, 0, 0, 0};
        for (int64_t r = c * gsz + part * 16; r < r1; r += 128) {
            uint32_t x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = (r + i < r1) ? __ldg(bits_t + (r + i) * Wp + w) : 0u;
            uint32_t ta, tb, fa, fb, ea, eb, sixteens;
            csa(ta, ones, ones, x[0], x[1]);
            csa(tb, ones, ones, x[2], x[3]);
            csa(fa, twos, twos, ta, tb);
            csa(ta, ones, ones, x[4], x[5]);
            csa(tb, ones, ones, x[6], x[7]);
            csa(fb, twos, twos, ta, tb);
            csa(ea, fours, fours, fa, fb);
            csa(ta, ones, ones, x[8], x[9]);
            csa(tb, ones, ones, x[10], x[11]);
            csa(fa, twos, twos, ta, tb);
            csa(ta, ones, ones, x[12], x[13]);
            csa(tb, ones, ones, x[14], x[15]);
            csa(fb, twos, twos, ta, tb);
            csa(eb, fours, fours, fa, fb);
            csa(sixteens, eights, eights, ea, eb);
            uint32_t carry = sixteens;
#pragma unroll
            for (int p = 0; p < 6; ++p) {
                const uint32_t tcar = hi[p] & carry;
                hi[p] ^= carry;
                carry = tcar;
            }
        }
        // sum the partial counts of the 8 partners sample by sample (every partner ends with all 32 sums
        // it needs: it writes samples part*4 .. part*4+3)
        int mine[4] = {0, 0, 0, 0};
#pragma unroll
        for (int src = 0; src < 8; ++src) {
            const int lane_src = (threadIdx.x & 24) | src;
            const uint32_t o1 = __shfl_sync(0xffffffffu, ones, lane_src), o2 = __shfl_sync(0xffffffffu, twos, lane_src);
            const uint32_t o4 = __shfl_sync(0xffffffffu, fours, lane_src), o8 = __shfl_sync(0xffffffffu, eights, lane_src);
            uint32_t oh[6];
#pragma unroll
            for (int p = 0; p < 6; ++p) oh[p] = __shfl_sync(0xffffffffu, hi[p], lane_src);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int s = part * 4 + q;
                int v = ((o1 >> s) & 1) | (((o2 >> s) & 1) << 1) | (((o4 >> s) & 1) << 2) | (((o8 >> s) & 1) << 3);
#pragma unroll
                for (int p = 0; p < 6; ++p) v |= ((oh[p] >> s) & 1) << (4 + p);
                mine[q] += v;
            }
        }
        if (live) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int64_t b = w * 32 + part * 4 + q;
                if (b < B) counts[b * k + c] = mine[q];
            }
        }
    }
}

}  // namespace

DL_EXPORT int dl_popcount_groupsum_t(const uint32_t* bits_t, int32_t* counts, int64_t N, int64_t k,
                                     int64_t B, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(bits_t && counts && N > 0 && k > 0 && B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    const int64_t gsz = dl_ceil_div(N, k);
    DL_REQUIRE(gsz < 1024);  // ten count planes
    const int64_t blocks = dl_min64(dl_ceil_div(k * (Bp / 32) * 8, 128), (int64_t)DL_NUM_SMS * 32);
    popcount_groupsum_kernel<<<(unsigned)blocks, 128, 0, dl_cast(stream)>>>(bits_t, counts, N, (int)k, gsz, B,
                                                                          Bp / 32);
    return dl_launch_status();
}
