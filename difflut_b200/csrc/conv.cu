// Patch extraction for the convolutional LUT layer and its adjoint.
//
// The reference extracts patches with nn.Unfold, transposes them to (batch*patches, C*kh*kw) rows and
// feeds them to its layers (difflut/layers/convolutional.py:194-205); the adjoint is autograd's fold.
// Here a "sample" is one patch s = b*P + p (p = oy*OW + ox) and a "feature" is f = (c*kh + ki)*kw + kj,
// the same order nn.Unfold uses.  Patches are produced directly in the layouts the LUT kernels read:
// fp32 rows (S, F), or thresholded and bit-packed feature-major [F][Bp/32], without an intermediate.
// Out-of-image taps (padding) read as 0.  The adjoints gather: one thread owns one input pixel and
// sums the taps that cover it, so there are no atomics and the sums have a fixed order.
#include "common.cuh"

namespace {

struct ConvGeom {
    int B, C, H, W;      // input (B, C, H, W)
    int kh, kw, sh, sw;  // receptive field, stride
    int ph, pw;          // zero padding
    int OH, OW;          // output positions
};

__host__ __device__ inline int64_t geom_patches(const ConvGeom& g) { return (int64_t)g.OH * g.OW; }

// fp32 rows: patches[s][f]
__global__ void unfold_rows_kernel(const float* __restrict__ x, float* __restrict__ patches, ConvGeom g) {
    const int F = g.C * g.kh * g.kw;
    const int64_t P = geom_patches(g);
    const int64_t total = (int64_t)g.B * P * F;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t s = t / F;
        const int f = (int)(t - s * F);
        const int b = (int)(s / P);
        const int p = (int)(s - (int64_t)b * P);
        const int oy = p / g.OW, ox = p - oy * g.OW;
        const int c = f / (g.kh * g.kw);
        const int r = f - c * g.kh * g.kw;
        const int ki = r / g.kw, kj = r - ki * g.kw;
        const int iy = oy * g.sh - g.ph + ki, ix = ox * g.sw - g.pw + kj;
        float v = 0.f;
        if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W)
            v = __ldg(x + (((int64_t)b * g.C + c) * g.H + iy) * g.W + ix);
        patches[t] = v;
    }
}

// Bit-packed feature-major.  A CTA owns 1024 consecutive samples (32 words): their patch origins go
// to shared memory once, then each warp walks features; for a feature it forms the 32 words with
// one ballot each and lane k keeps word k, so every feature row gets one coalesced 128-byte store.
constexpr int UNF_WORDS = 32;
constexpr int UNF_SAMPLES = UNF_WORDS * 32;

__global__ void __launch_bounds__(256)
unfold_pack_t_kernel(const float* __restrict__ x, uint32_t* __restrict__ bits_t, ConvGeom g, float threshold,
                     int64_t S, int64_t Wp) {
    __shared__ int32_t base[UNF_SAMPLES];  // offset of (b, c=0, iy0, ix0) in x; may point outside the image
    __shared__ int16_t oy0[UNF_SAMPLES], ox0[UNF_SAMPLES];
    const int F = g.C * g.kh * g.kw;
    const int64_t P = geom_patches(g);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t s0 = (int64_t)blockIdx.x * UNF_SAMPLES;
    for (int k = threadIdx.x; k < UNF_SAMPLES; k += blockDim.x) {
        const int64_t s = s0 + k;
        if (s < S) {
            const int b = (int)(s / P);
            const int p = (int)(s - (int64_t)b * P);
            const int oy = p / g.OW, ox = p - oy * g.OW;
            const int iy = oy * g.sh - g.ph, ix = ox * g.sw - g.pw;
            oy0[k] = (int16_t)iy;
            ox0[k] = (int16_t)ix;
            base[k] = (b * g.C * g.H + iy) * g.W + ix;
        } else {
            oy0[k] = (int16_t)-30000;  // every tap out of range: padding samples pack as 0
            ox0[k] = (int16_t)-30000;
            base[k] = 0;
        }
    }
    __syncthreads();
    const int64_t w0 = (int64_t)blockIdx.x * UNF_WORDS;
    for (int f = warp; f < F; f += 8) {
        const int c = f / (g.kh * g.kw);
        const int r = f - c * g.kh * g.kw;
        const int ki = r / g.kw, kj = r - ki * g.kw;
        const int off = (c * g.H + ki) * g.W + kj;
        uint32_t mine = 0;
#pragma unroll 4
        for (int k = 0; k < UNF_WORDS; ++k) {
            const int idx = k * 32 + lane;
            const int iy = oy0[idx] + ki, ix = ox0[idx] + kj;
            bool bit = false;
            if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) bit = __ldg(x + base[idx] + off) >= threshold;
            const uint32_t word = __ballot_sync(0xffffffffu, bit);
            if (lane == k) mine = word;
        }
        if (w0 + lane < Wp) bits_t[(int64_t)f * Wp + w0 + lane] = mine;
    }
}

// Adjoint: gx[b,c,iy,ix] = sum over taps (ki,kj) and positions (oy,ox) with oy*sh - ph + ki == iy, ... of
// the patch gradient.  T_LAYOUT: src is feature-major [F][ld] (ld = padded sample count), else rows (S, F).
template <bool T_LAYOUT>
__global__ void fold_kernel(const float* __restrict__ src, float* __restrict__ gx, ConvGeom g, int64_t ld) {
    const int F = g.C * g.kh * g.kw;
    const int64_t P = geom_patches(g);
    const int64_t total = (int64_t)g.B * g.C * g.H * g.W;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int ix = (int)(t % g.W);
        int64_t q = t / g.W;
        const int iy = (int)(q % g.H);
        q /= g.H;
        const int c = (int)(q % g.C);
        const int b = (int)(q / g.C);
        float acc = 0.f;
        for (int ki = 0; ki < g.kh; ++ki) {
            const int ty = iy + g.ph - ki;
            if (ty < 0 || ty % g.sh != 0) continue;
            const int oy = ty / g.sh;
            if (oy >= g.OH) continue;
            for (int kj = 0; kj < g.kw; ++kj) {
                const int tx = ix + g.pw - kj;
                if (tx < 0 || tx % g.sw != 0) continue;
                const int ox = tx / g.sw;
                if (ox >= g.OW) continue;
                const int f = (c * g.kh + ki) * g.kw + kj;
                const int64_t s = (int64_t)b * P + (int64_t)oy * g.OW + ox;
                acc += T_LAYOUT ? __ldg(src + (int64_t)f * ld + s) : __ldg(src + s * F + f);
            }
        }
        gx[t] = acc;
    }
}

int make_geom(ConvGeom& g, int64_t B, int64_t C, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t sh,
              int64_t sw, int64_t ph, int64_t pw) {
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
        return DL_ERR_ARG;
    if (H + 2 * ph < kh || W + 2 * pw < kw) return DL_ERR_ARG;
    if (H > 16384 || W > 16384 || kh > 1024 || kw > 1024 || ph > 1024 || pw > 1024) return DL_ERR_TOO_LARGE;
    if (B * C * H * W >= ((int64_t)1 << 31)) return DL_ERR_TOO_LARGE;  // 32-bit pixel offsets in the pack kernel
    g.B = (int)B; g.C = (int)C; g.H = (int)H; g.W = (int)W;
    g.kh = (int)kh; g.kw = (int)kw; g.sh = (int)sh; g.sw = (int)sw; g.ph = (int)ph; g.pw = (int)pw;
    g.OH = (int)((H + 2 * ph - kh) / sh + 1);
    g.OW = (int)((W + 2 * pw - kw) / sw + 1);
    return DL_OK;
}

}  // namespace

DL_EXPORT int64_t dl_unfold_positions(int64_t size, int64_t k, int64_t stride, int64_t pad) {
    if (size <= 0 || k <= 0 || stride <= 0 || pad < 0 || size + 2 * pad < k) return 0;
    return (size + 2 * pad - k) / stride + 1;
}

DL_EXPORT int dl_unfold_rows(const float* x, float* patches, int64_t B, int64_t C, int64_t H, int64_t W,
                             int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                             dl_stream_t stream) {
    DL_REQUIRE(x && patches);
    ConvGeom g;
    const int rc = make_geom(g, B, C, H, W, kh, kw, sh, sw, ph, pw);
    if (rc != DL_OK) return rc;
    const int64_t total = B * geom_patches(g) * C * kh * kw;
    const int64_t blocks = dl_min64(dl_ceil_div(total, 256), (int64_t)DL_NUM_SMS * 16);
    unfold_rows_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(x, patches, g);
    return dl_launch_status();
}

DL_EXPORT int dl_unfold_pack_t(const float* x, uint32_t* bits_t, int64_t B, int64_t C, int64_t H, int64_t W,
                               int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                               float threshold, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(x && bits_t && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    ConvGeom g;
    const int rc = make_geom(g, B, C, H, W, kh, kw, sh, sw, ph, pw);
    if (rc != DL_OK) return rc;
    const int64_t S = B * geom_patches(g);
    DL_REQUIRE(Bp >= S);
    const int64_t Wp = Bp / 32;
    const int64_t blocks = dl_ceil_div(Wp, UNF_WORDS);
    if (blocks > 0x7fffffff) return DL_ERR_TOO_LARGE;
    unfold_pack_t_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(x, bits_t, g, threshold, S, Wp);
    return dl_launch_status();
}

DL_EXPORT int dl_fold_rows(const float* gpatches, float* gx, int64_t B, int64_t C, int64_t H, int64_t W,
                           int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw,
                           dl_stream_t stream) {
    DL_REQUIRE(gpatches && gx);
    ConvGeom g;
    const int rc = make_geom(g, B, C, H, W, kh, kw, sh, sw, ph, pw);
    if (rc != DL_OK) return rc;
    const int64_t blocks = dl_min64(dl_ceil_div(B * C * H * W, 256), (int64_t)DL_NUM_SMS * 16);
    fold_kernel<false><<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(gpatches, gx, g, 0);
    return dl_launch_status();
}

DL_EXPORT int dl_fold_t(const float* gpatches_t, float* gx, int64_t B, int64_t C, int64_t H, int64_t W,
                        int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t Bp,
                        dl_stream_t stream) {
    DL_REQUIRE(gpatches_t && gx && Bp > 0);
    ConvGeom g;
    const int rc = make_geom(g, B, C, H, W, kh, kw, sh, sw, ph, pw);
    if (rc != DL_OK) return rc;
    DL_REQUIRE(Bp >= B * geom_patches(g));
    const int64_t blocks = dl_min64(dl_ceil_div(B * C * H * W, 256), (int64_t)DL_NUM_SMS * 16);
    fold_kernel<true><<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(gpatches_t, gx, g, Bp);
    return dl_launch_status();
}
