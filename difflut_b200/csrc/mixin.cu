// Training-time options of a LUT layer (difflut/layers/base_layer.py:149-339) as kernels:
//   * bit-flip augmentation: every input is replaced by 1 - x with probability p, without gradient.  For
//     fp32 rows this is an elementwise pass; for bit-packed feature-major activations it is an XOR with a
//     Bernoulli(p) mask, applied right after packing, so a convolution never materialises its patches.
//     The random bits come from a counter-based generator (a 64-bit mix of seed and element index): the
//     result depends only on (seed, position), not on the launch geometry.
//   * gradient rescaling: (g - mean) * sqrt(target / (mean((g - mean)^2) + eps)) over the whole layer
//     gradient or per sample; sums are accumulated in double in a fixed order (reproducible).
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t mix_u32(uint64_t seed, uint64_t index) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (index + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (uint32_t)(z >> 32);
}

__global__ void flip_rows_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t count,
                                 uint32_t threshold, uint64_t seed) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        out[i] = mix_u32(seed, (uint64_t)i) < threshold ? 1.0f - v : v;
    }
}

// element index of bit b of row f = f * B + b: the same elements flip as flip_rows_kernel would flip on
// the (F, B) feature-major matrix, whatever the padding
__global__ void bits_flip_t_kernel(uint32_t* __restrict__ bits_t, int64_t F, int64_t B, int64_t Wp,
                                   uint32_t threshold, uint64_t seed) {
    const int64_t total = F * Wp;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t f = t / Wp, w = t - f * Wp;
        uint32_t mask = 0;
#pragma unroll 8
        for (int k = 0; k < 32; ++k) {
            const int64_t b = w * 32 + k;
            if (b < B && mix_u32(seed, (uint64_t)(f * B + b)) < threshold) mask |= 1u << k;
        }
        if (mask != 0) bits_t[t] ^= mask;
    }
}

// Exact-count variant (the reference's choice below p = 0.05, base_layer.py:226-262): the caller draws the
// positions (a random permutation's first `flips` entries, so they are distinct) and these kernels apply them.
__global__ void copy_f32_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t count) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = x[i];
}

__global__ void flip_at_kernel(const float* __restrict__ x, float* __restrict__ out, const int64_t* __restrict__ idx,
                               int64_t count, int64_t flips) {
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < flips;
         k += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = idx[k];
        if (i >= 0 && i < count) out[i] = 1.0f - x[i];
    }
}

// position e of the row-major (B, F) matrix = sample e / F, feature e % F; two positions can share a word
__global__ void bits_flip_at_t_kernel(uint32_t* __restrict__ bits_t, const int64_t* __restrict__ idx, int64_t flips,
                                      int64_t F, int64_t B, int64_t Wp) {
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < flips;
         k += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = idx[k];
        if (e < 0 || e >= F * B) continue;
        const int64_t b = e / F, f = e - b * F;
        atomicXor(bits_t + f * Wp + (b >> 5), 1u << (b & 31));
    }
}

__device__ __forceinline__ double block_sum(double v, double* shared) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    __syncthreads();
    if (lane == 0) shared[warp] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += shared[w];
    return total;
}

// one CTA per row
__global__ void __launch_bounds__(256)
rescale_rows_kernel(const float* __restrict__ g, float* __restrict__ out, int64_t cols, float target,
                    int subtract_mean, float eps) {
    __shared__ double red[8];
    const float* row = g + (int64_t)blockIdx.x * cols;
    float* dst = out + (int64_t)blockIdx.x * cols;
    double mean = 0.0;
    if (subtract_mean) {
        double s = 0.0;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += (double)row[c];
        mean = block_sum(s, red) / (double)cols;
    }
    double q = 0.0;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const double d = (double)row[c] - mean;
        q += d * d;
    }
    const double var = block_sum(q, red) / (double)cols;
    const float scale = sqrtf(target / ((float)var + eps));
    const float mu = (float)mean;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = (row[c] - mu) * scale;
}

// whole tensor: per-CTA partial sums of g and g^2 (double), then every CTA folds the partial list
constexpr int RESCALE_BLOCKS = 592;

__global__ void __launch_bounds__(256)
rescale_partial_kernel(const float* __restrict__ g, double* __restrict__ partial, int64_t count) {
    __shared__ double red[8];
    double s = 0.0, q = 0.0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x) {
        const double v = (double)g[i];
        s += v;
        q += v * v;
    }
    const double ts = block_sum(s, red);
    const double tq = block_sum(q, red);
    if (threadIdx.x == 0) {
        partial[2 * blockIdx.x] = ts;
        partial[2 * blockIdx.x + 1] = tq;
    }
}

__global__ void __launch_bounds__(256)
rescale_apply_kernel(const float* __restrict__ g, float* __restrict__ out, const double* __restrict__ partial,
                     int nparts, int64_t count, float target, int subtract_mean, float eps) {
    double s = 0.0, q = 0.0;
    for (int p = 0; p < nparts; ++p) {  // same order in every thread
        s += partial[2 * p];
        q += partial[2 * p + 1];
    }
    const double mean = subtract_mean ? s / (double)count : 0.0;
    // mean((g - mean)^2) = mean(g^2) - 2 mean mean(g) + mean^2
    const double var = q / (double)count - 2.0 * mean * (s / (double)count) + mean * mean;
    const float scale = sqrtf(target / ((float)var + eps));
    const float mu = (float)mean;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (g[i] - mu) * scale;
}

uint32_t flip_threshold(float p) {
    if (p >= 1.0f) return 0xFFFFFFFFu;
    const double t = (double)p * 4294967296.0;
    return t <= 0.0 ? 0u : (uint32_t)t;
}

}  // namespace

DL_EXPORT int dl_flip_rows(const float* x, float* out, int64_t count, float probability, int64_t seed,
                           dl_stream_t stream) {
    DL_REQUIRE(x && out && count > 0 && probability >= 0.f && probability <= 1.f);
    const int64_t blocks = dl_min64(dl_ceil_div(count, 256), (int64_t)DL_NUM_SMS * 16);
    flip_rows_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(x, out, count, flip_threshold(probability), (uint64_t)seed);
    return dl_launch_status();
}

DL_EXPORT int dl_bits_flip_t(uint32_t* bits_t, int64_t F, int64_t B, int64_t Bp, float probability, int64_t seed,
                             dl_stream_t stream) {
    DL_REQUIRE(bits_t && F > 0 && B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE(probability >= 0.f && probability <= 1.f);
    const int64_t blocks = dl_min64(dl_ceil_div(F * (Bp / 32), 256), (int64_t)DL_NUM_SMS * 16);
    bits_flip_t_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(bits_t, F, B, Bp / 32,
                                                                     flip_threshold(probability), (uint64_t)seed);
    return dl_launch_status();
}

DL_EXPORT int dl_flip_at(const float* x, float* out, const int64_t* positions, int64_t count, int64_t flips,
                         dl_stream_t stream) {
    DL_REQUIRE(x && out && x != out && count > 0 && flips >= 0 && (positions || flips == 0));
    cudaStream_t s = dl_cast(stream);
    copy_f32_kernel<<<(unsigned)dl_min64(dl_ceil_div(count, 256), (int64_t)DL_NUM_SMS * 16), 256, 0, s>>>(x, out, count);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    if (flips > 0)
        flip_at_kernel<<<(unsigned)dl_min64(dl_ceil_div(flips, 256), (int64_t)DL_NUM_SMS * 16), 256, 0, s>>>(
            x, out, positions, count, flips);
    return dl_launch_status();
}

DL_EXPORT int dl_bits_flip_at_t(uint32_t* bits_t, const int64_t* positions, int64_t flips, int64_t F, int64_t B,
                                int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(bits_t && F > 0 && B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0 && flips >= 0 && (positions || flips == 0));
    if (flips > 0)
        bits_flip_at_t_kernel<<<(unsigned)dl_min64(dl_ceil_div(flips, 256), (int64_t)DL_NUM_SMS * 16), 256, 0,
                                dl_cast(stream)>>>(bits_t, positions, flips, F, B, Bp / 32);
    return dl_launch_status();
}

DL_EXPORT int64_t dl_grad_rescale_scratch_doubles(void) { return 2 * RESCALE_BLOCKS; }

DL_EXPORT int dl_grad_rescale(const float* g, float* out, int64_t rows, int64_t cols, int per_row, float target_std,
                              int subtract_mean, float eps, double* scratch, dl_stream_t stream) {
    DL_REQUIRE(g && out && rows > 0 && cols > 0 && target_std > 0.f && eps > 0.f);
    if (per_row) {
        DL_REQUIRE(rows <= 0x7fffffff);
        rescale_rows_kernel<<<(unsigned)rows, 256, 0, dl_cast(stream)>>>(g, out, cols, target_std, subtract_mean, eps);
        return dl_launch_status();
    }
    DL_REQUIRE(scratch);
    const int64_t count = rows * cols;
    const int nparts = (int)dl_min64(dl_ceil_div(count, 256), RESCALE_BLOCKS);
    rescale_partial_kernel<<<nparts, 256, 0, dl_cast(stream)>>>(g, scratch, count);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    rescale_apply_kernel<<<nparts, 256, 0, dl_cast(stream)>>>(g, out, scratch, nparts, count, target_std,
                                                             subtract_mean, eps);
    return dl_launch_status();
}
