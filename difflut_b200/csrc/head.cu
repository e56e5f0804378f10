// GroupSum, cross-entropy and Adam: the small kernels after the last LUT layer.
#include "common.cuh"

namespace {

// rows: one warp per (sample, class); lanes stride over the class's contiguous columns.
__global__ void groupsum_rows_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t B,
                                     int64_t F, int k, int64_t gsz, float inv_tau) {
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < B * k; w += nwarps) {
        const int64_t b = w / k, c = w - b * k;
        const int64_t c0 = c * gsz;
        int64_t c1 = c0 + gsz;
        if (c1 > F) c1 = F;
        float acc = 0.f;
        for (int64_t col = c0 + lane; col < c1; col += 32) acc += x[b * F + col];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) out[w] = acc * inv_tau;
    }
}

__global__ void groupsum_rows_bwd_kernel(const float* __restrict__ gout, float* __restrict__ gx,
                                         int64_t B, int64_t F, int k, int64_t gsz, float inv_tau) {
    const int64_t total = B * F;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t / F, col = t - b * F;
        gx[t] = gout[b * k + col / gsz] * inv_tau;
    }
}

// feature-major: thread per (class, sample); rows of the class are read coalesced.
__global__ void groupsum_t_kernel(const float* __restrict__ vals_t, float* __restrict__ logits_t,
                                  int64_t F, int k, int64_t gsz, float inv_tau, int64_t Bp) {
    const int64_t total = (int64_t)k * Bp;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = t / Bp, b = t - c * Bp;
        int64_t r1 = (c + 1) * gsz;
        if (r1 > F) r1 = F;
        float acc = 0.f;
        for (int64_t r = c * gsz; r < r1; ++r) acc += vals_t[r * Bp + b];
        logits_t[t] = acc * inv_tau;
    }
}

// softmax cross-entropy, thread per sample
__global__ void ce_t_kernel(const float* __restrict__ logits_t, const int32_t* __restrict__ labels,
                            float* __restrict__ dlogits_t, float* __restrict__ loss_rows, int64_t B,
                            float inv_bg, int k, int64_t Bp) {
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < Bp;
         b += (int64_t)gridDim.x * blockDim.x) {
        if (b >= B) {
            for (int c = 0; c < k; ++c) dlogits_t[c * Bp + b] = 0.f;
            loss_rows[b] = 0.f;
            continue;
        }
        float mx = -INFINITY;
        for (int c = 0; c < k; ++c) mx = fmaxf(mx, logits_t[c * Bp + b]);
        float sum = 0.f;
        for (int c = 0; c < k; ++c) sum += expf(logits_t[c * Bp + b] - mx);
        const float lse = mx + logf(sum);
        const int y = labels[b];
        if (y < 0 || y >= k) {
            // no such class (torch's cross_entropy raises for it): the row gets no gradient and a NaN loss,
            // which shows in the step's loss instead of reading outside the logits
            for (int c = 0; c < k; ++c) dlogits_t[c * Bp + b] = 0.f;
            loss_rows[b] = __int_as_float(0x7fc00000);
            continue;
        }
        const float inv = 1.0f / sum;
        for (int c = 0; c < k; ++c) {
            const float p = expf(logits_t[c * Bp + b] - mx) * inv;
            dlogits_t[c * Bp + b] = (p - (c == y ? 1.f : 0.f)) * inv_bg;
        }
        loss_rows[b] = lse - logits_t[(int64_t)y * Bp + b];
    }
}

// single CTA, fixed-order tree: reproducible
__global__ void __launch_bounds__(1024)
loss_sum_kernel(const float* __restrict__ loss_rows, float* __restrict__ loss, int64_t Bp, float inv_bg) {
    __shared__ double part[1024];
    double acc = 0.0;
    for (int64_t b = threadIdx.x; b < Bp; b += 1024) acc += (double)loss_rows[b];
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = 512; s > 0; s >>= 1) {
        if (threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) loss[0] = (float)(part[0] * (double)inv_bg);
}

__global__ void adam_advance_kernel(double* state, double b1, double b2) {
    state[0] *= b1;
    state[1] *= b2;
}

// four elements per thread (16-byte accesses); the tail is handled element-wise
__global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                            float* __restrict__ v, const double* __restrict__ state, int64_t count,
                            float lr, float b1, float b2, float eps, float gscale) {
    // bias corrections in double, as the host-side optimiser computes them
    const double bc1 = 1.0 - state[0];
    const double bc2 = 1.0 - state[1];
    const float step_size = (float)((double)lr / bc1);
    const float bc2_sqrt = (float)sqrt(bc2);
    const int64_t quads = count >> 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads;
         i += (int64_t)gridDim.x * blockDim.x) {
        float4 pp = reinterpret_cast<float4*>(p)[i], mm = reinterpret_cast<float4*>(m)[i];
        float4 vv = reinterpret_cast<float4*>(v)[i];
        const float4 gg = reinterpret_cast<const float4*>(g)[i];
        pp.x = adam_update(pp.x, gg.x, gscale, mm.x, vv.x, step_size, bc2_sqrt, b1, b2, eps);
        pp.y = adam_update(pp.y, gg.y, gscale, mm.y, vv.y, step_size, bc2_sqrt, b1, b2, eps);
        pp.z = adam_update(pp.z, gg.z, gscale, mm.z, vv.z, step_size, bc2_sqrt, b1, b2, eps);
        pp.w = adam_update(pp.w, gg.w, gscale, mm.w, vv.w, step_size, bc2_sqrt, b1, b2, eps);
        reinterpret_cast<float4*>(p)[i] = pp;
        reinterpret_cast<float4*>(m)[i] = mm;
        reinterpret_cast<float4*>(v)[i] = vv;
    }
    for (int64_t i = (quads << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x)
        p[i] = adam_update(p[i], g[i], gscale, m[i], v[i], step_size, bc2_sqrt, b1, b2, eps);
}

// Adam step whose gradient is the ordered sum of `groups` partial-gradient slabs; the summed
// gradient is also written to g_out (it is the .grad users read)
__global__ void adam_groups_kernel(float* __restrict__ p, const float* __restrict__ partial, int64_t stride,
                                   int groups, float* __restrict__ g_out, float* __restrict__ m,
                                   float* __restrict__ v, const double* __restrict__ state, int64_t count, float lr,
                                   float b1, float b2, float eps, float gscale) {
    const double bc1 = 1.0 - state[0];
    const double bc2 = 1.0 - state[1];
    const float step_size = (float)((double)lr / bc1);
    const float bc2_sqrt = (float)sqrt(bc2);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int g = 0; g < groups; ++g) acc += partial[(int64_t)g * stride + i];
        g_out[i] = acc;
        float mi = m[i], vi = v[i];
        p[i] = adam_update(p[i], acc, gscale, mi, vi, step_size, bc2_sqrt, b1, b2, eps);
        m[i] = mi;
        v[i] = vi;
    }
}

}  // namespace

DL_EXPORT int dl_groupsum_rows(const float* x, float* out, int64_t B, int64_t F, int64_t k, float tau,
                               dl_stream_t stream) {
    DL_REQUIRE(x && out && B > 0 && F > 0 && k > 0 && tau > 0.f);
    const int64_t gsz = dl_ceil_div(F, k);
    const int64_t blocks = dl_min64(dl_ceil_div(B * k * 32, 256), (int64_t)DL_NUM_SMS * 32);
    groupsum_rows_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(x, out, B, F, (int)k, gsz, 1.0f / tau);
    return dl_launch_status();
}

DL_EXPORT int dl_groupsum_rows_bwd(const float* gout, float* gx, int64_t B, int64_t F, int64_t k,
                                   float tau, dl_stream_t stream) {
    DL_REQUIRE(gout && gx && B > 0 && F > 0 && k > 0 && tau > 0.f);
    const int64_t gsz = dl_ceil_div(F, k);
    const int64_t blocks = dl_min64(dl_ceil_div(B * F, 256), (int64_t)DL_NUM_SMS * 32);
    groupsum_rows_bwd_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(gout, gx, B, F, (int)k, gsz,
                                                                          1.0f / tau);
    return dl_launch_status();
}

DL_EXPORT int dl_groupsum_t(const float* vals_t, float* logits_t, int64_t F, int64_t k, float tau,
                            int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(vals_t && logits_t && F > 0 && k > 0 && tau > 0.f && Bp > 0);
    const int64_t gsz = dl_ceil_div(F, k);
    const int64_t blocks = dl_min64(dl_ceil_div(k * Bp, 128), (int64_t)DL_NUM_SMS * 32);
    groupsum_t_kernel<<<(unsigned)blocks, 128, 0, dl_cast(stream)>>>(vals_t, logits_t, F, (int)k, gsz,
                                                                   1.0f / tau, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_ce_t(const float* logits_t, const int32_t* labels, float* dlogits_t, float* loss_rows,
                      float* loss, int64_t B, int64_t B_global, int64_t k, int64_t Bp,
                      dl_stream_t stream) {
    DL_REQUIRE(logits_t && labels && dlogits_t && loss_rows);
    DL_REQUIRE(B > 0 && B_global >= B && k > 0 && Bp >= B);
    const float inv_bg = (float)(1.0 / (double)B_global);
    const int64_t blocks = dl_min64(dl_ceil_div(Bp, 128), (int64_t)DL_NUM_SMS * 8);
    ce_t_kernel<<<(unsigned)blocks, 128, 0, dl_cast(stream)>>>(logits_t, labels, dlogits_t, loss_rows, B,
                                                             inv_bg, (int)k, Bp);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    if (loss != nullptr) loss_sum_kernel<<<1, 1024, 0, dl_cast(stream)>>>(loss_rows, loss, Bp, inv_bg);
    return dl_launch_status();
}

DL_EXPORT int dl_loss_sum(const float* loss_rows, float* loss, int64_t B_global, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(loss_rows && loss && B_global > 0 && Bp > 0);
    loss_sum_kernel<<<1, 1024, 0, dl_cast(stream)>>>(loss_rows, loss, Bp, (float)(1.0 / (double)B_global));
    return dl_launch_status();
}

DL_EXPORT int dl_adam_step(float* p, const float* g, float* m, float* v, double* state, int64_t count,
                           float lr, float beta1, float beta2, float eps, float gscale,
                           dl_stream_t stream) {
    DL_REQUIRE(p && g && m && v && state && count > 0);
    DL_REQUIRE_ALIGNED(p, 16);
    DL_REQUIRE_ALIGNED(g, 16);
    DL_REQUIRE_ALIGNED(m, 16);
    DL_REQUIRE_ALIGNED(v, 16);
    adam_advance_kernel<<<1, 1, 0, dl_cast(stream)>>>(state, (double)beta1, (double)beta2);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    const int64_t blocks = dl_min64(dl_ceil_div(dl_ceil_div(count, 4), 256), (int64_t)DL_NUM_SMS * 16);
    adam_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(p, g, m, v, state, count, lr, beta1, beta2,
                                                             eps, gscale);
    return dl_launch_status();
}

DL_EXPORT int dl_adam_advance(double* state, float beta1, float beta2, dl_stream_t stream) {
    DL_REQUIRE(state);
    adam_advance_kernel<<<1, 1, 0, dl_cast(stream)>>>(state, (double)beta1, (double)beta2);
    return dl_launch_status();
}

DL_EXPORT int dl_adam_apply(float* p, const float* g, float* m, float* v, const double* state, int64_t count,
                            float lr, float beta1, float beta2, float eps, float gscale, dl_stream_t stream) {
    DL_REQUIRE(p && g && m && v && state && count > 0);
    DL_REQUIRE_ALIGNED(p, 16);
    DL_REQUIRE_ALIGNED(g, 16);
    DL_REQUIRE_ALIGNED(m, 16);
    DL_REQUIRE_ALIGNED(v, 16);
    const int64_t blocks = dl_min64(dl_ceil_div(dl_ceil_div(count, 4), 256), (int64_t)DL_NUM_SMS * 16);
    adam_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(p, g, m, v, state, count, lr, beta1, beta2,
                                                             eps, gscale);
    return dl_launch_status();
}

DL_EXPORT int dl_adam_step_groups(float* p, const float* partial, int64_t stride, int64_t groups, float* g_out,
                                  float* m, float* v, double* state, int64_t count, float lr, float beta1,
                                  float beta2, float eps, float gscale, dl_stream_t stream) {
    DL_REQUIRE(p && partial && g_out && m && v && state && count > 0 && groups > 0 && stride >= count);
    adam_advance_kernel<<<1, 1, 0, dl_cast(stream)>>>(state, (double)beta1, (double)beta2);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    const int64_t blocks = dl_min64(dl_ceil_div(count, 256), (int64_t)DL_NUM_SMS * 16);
    adam_groups_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(p, partial, stride, (int)groups, g_out, m, v,
                                                                    state, count, lr, beta1, beta2, eps, gscale);
    return dl_launch_status();
}

DL_EXPORT int dl_version(void) { return 100; }

DL_EXPORT const char* dl_error_string(int code) {
    switch (code) {
        case DL_OK: return "ok";
        case DL_ERR_ARG: return "invalid argument (null pointer or inconsistent sizes)";
        case DL_ERR_UNSUPPORTED: return "unsupported node input count for this entry point";
        case DL_ERR_LAUNCH: return "CUDA reported an error at kernel launch";
        case DL_ERR_ALIGN: return "pointer or stride is not aligned as documented";
        case DL_ERR_TOO_LARGE: return "size exceeds a documented fixed capacity";
        default: return "unknown error code";
    }
}

DL_EXPORT int64_t dl_padded_batch(int64_t B) {
    return B <= 0 ? 0 : dl_ceil_div(B, DL_BATCH_ALIGN) * DL_BATCH_ALIGN;
}
