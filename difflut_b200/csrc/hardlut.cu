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

// Thread per (class, word of 32 samples).  The class's rows are added bit-sliced: 16 rows at a time
// go through a carry-save adder tree into the planes ones / twos / fours / eights, the resulting
// sixteens word is rippled into six higher planes; at the end the planes are read out per sample.
// About 3 logic ops per row and word instead of 3 per row and SAMPLE.
__global__ void __launch_bounds__(128)
popcount_groupsum_kernel(const uint32_t* __restrict__ bits_t, int32_t* __restrict__ counts, int64_t N, int k,
                         int64_t gsz, int64_t B, int64_t Wp) {
    const int64_t total = (int64_t)k * Wp;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = t / Wp, w = t - c * Wp;
        if (w * 32 >= B) continue;
        int64_t r1 = (c + 1) * gsz;
        if (r1 > N) r1 = N;
        uint32_t ones = 0, twos = 0, fours = 0, eights = 0, hi[6] = {0, 0, 0, 0, 0, 0};
        for (int64_t r = c * gsz; r < r1; r += 16) {
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
#pragma unroll 4
        for (int s = 0; s < 32; ++s) {
            const int64_t b = w * 32 + s;
            if (b >= B) break;
            int v = ((ones >> s) & 1) | (((twos >> s) & 1) << 1) | (((fours >> s) & 1) << 2) | (((eights >> s) & 1) << 3);
#pragma unroll
            for (int p = 0; p < 6; ++p) v |= ((hi[p] >> s) & 1) << (4 + p);
            counts[b * k + c] = v;
        }
    }
}

}  // namespace

DL_EXPORT int dl_popcount_groupsum_t(const uint32_t* bits_t, int32_t* counts, int64_t N, int64_t k,
                                     int64_t B, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(bits_t && counts && N > 0 && k > 0 && B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    const int64_t gsz = dl_ceil_div(N, k);
    DL_REQUIRE(gsz < 1024);  // ten count planes
    const int64_t blocks = dl_min64(dl_ceil_div(k * (Bp / 32), 128), (int64_t)DL_NUM_SMS * 32);
    popcount_groupsum_kernel<<<(unsigned)blocks, 128, 0, dl_cast(stream)>>>(bits_t, counts, N, (int)k, gsz, B,
                                                                          Bp / 32);
    return dl_launch_status();
}
