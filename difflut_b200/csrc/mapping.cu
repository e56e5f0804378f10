// RandomLayer gather on fp32 rows and its scatter-add backward (API-exact `get_mapping`).
//
// Forward is an indexed copy.  The backward replaces the reference's global fp32 atomics
// (difflut/layers/cuda/mapping_cuda_kernel.cu:136-162) by a segmented sum over the inverse map:
// the owner of (b, f) adds the gradient columns listed for feature f in a fixed order.  The forward has a plain
// form (one thread per element) and a shared-memory staged form that the entry point prefers when a row fits;
// both are exact copies.  A staged backward (gradient row walked in shared-memory tiles) was measured slower
// than the plain one at the first layer's width (0.92 vs 0.78 ms for 2048 rows) and is not kept.
#include "common.cuh"

namespace {

__global__ void gather_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ map,
                                   float* __restrict__ out, int64_t B, int64_t F, int64_t M) {
    const int64_t total = B * M;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t / M, c = t - b * M;
        out[t] = __ldg(x + b * F + __ldg(map + c));
    }
}

// Thread (row group, f): four rows share one walk over f's entry list, so an index is loaded once per four
// gradients and four independent gradient loads are in flight per entry.
constexpr int BWD_ROWS = 4;

__global__ void gather_rows_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ inv_ptr,
                                       const int32_t* __restrict__ inv_ent, float* __restrict__ gx,
                                       int64_t B, int64_t F, int64_t M) {
    const int64_t groups = (B + BWD_ROWS - 1) / BWD_ROWS;
    const int64_t total = groups * F;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t bg = t / F, f = t - bg * F;
        const int64_t b0 = bg * BWD_ROWS;
        const int e0 = __ldg(inv_ptr + f), e1 = __ldg(inv_ptr + f + 1);
        float acc[BWD_ROWS];
#pragma unroll
        for (int r = 0; r < BWD_ROWS; ++r) acc[r] = 0.f;
        for (int e = e0; e < e1; ++e) {
            const int64_t c = __ldg(inv_ent + e);
#pragma unroll
            for (int r = 0; r < BWD_ROWS; ++r)
                if (b0 + r < B) acc[r] += __ldg(g + (b0 + r) * M + c);
        }
#pragma unroll
        for (int r = 0; r < BWD_ROWS; ++r)
            if (b0 + r < B) gx[(b0 + r) * F + f] = acc[r];
    }
}

// Shared-memory staged forward.  One CTA works on one sample row at a time: the row x[b, :] (F floats) is copied into shared memory with coalesced 16-byte loads; every
// output element is then a shared-memory read at a mapped position and the (B, M) output leaves as
// coalesced 16-byte stores.  HBM sees each input once and each output once.
constexpr int STAGE_THREADS = 512;

__global__ void __launch_bounds__(STAGE_THREADS)
gather_rows_staged_kernel(const float* __restrict__ x, const int32_t* __restrict__ map, float* __restrict__ out,
                          int64_t B, int64_t F, int64_t M) {
    extern __shared__ float row_s[];
    const bool vec_in = (F & 3) == 0, vec_out = (M & 3) == 0;
    for (int64_t b = blockIdx.x; b < B; b += gridDim.x) {
        __syncthreads();  // the previous row is no longer read
        const float* xr = x + b * F;
        if (vec_in) {
            for (int64_t q = threadIdx.x; q < (F >> 2); q += STAGE_THREADS)
                reinterpret_cast<float4*>(row_s)[q] = __ldg(reinterpret_cast<const float4*>(xr) + q);
        } else {
            for (int64_t f = threadIdx.x; f < F; f += STAGE_THREADS) row_s[f] = __ldg(xr + f);
        }
        __syncthreads();
        float* orow = out + b * M;
        if (vec_out) {
            for (int64_t q = threadIdx.x; q < (M >> 2); q += STAGE_THREADS) {
                const int4 m = __ldg(reinterpret_cast<const int4*>(map) + q);
                reinterpret_cast<float4*>(orow)[q] = make_float4(row_s[m.x], row_s[m.y], row_s[m.z], row_s[m.w]);
            }
        } else {
            for (int64_t c = threadIdx.x; c < M; c += STAGE_THREADS) orow[c] = row_s[__ldg(map + c)];
        }
    }
}

constexpr int64_t STAGE_SMEM_BUDGET = 220 * 1024;  // bytes of dynamic shared memory a staged kernel may ask for

}  // namespace

DL_EXPORT int dl_gather_rows(const float* x, const int32_t* map, float* out, int64_t B, int64_t F,
                             int64_t N, int64_t n, dl_stream_t stream) {
    DL_REQUIRE(x && map && out && B > 0 && F > 0 && N > 0 && n > 0);
    const int64_t M = N * n;
    const bool aligned = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(map) % 16 == 0;
    if (aligned && F * 4 <= STAGE_SMEM_BUDGET && M >= 1024) {
        // a row of inputs fits shared memory: staged kernel, one row per CTA at a time
        const size_t smem = (size_t)F * 4;
        if (cudaFuncSetAttribute(gather_rows_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) ==
            cudaSuccess) {
            const int64_t per_sm = dl_min64(4, (int64_t)(220 * 1024) / (int64_t)(smem + 1024));
            const int64_t blocks = dl_min64(B, (int64_t)DL_NUM_SMS * (per_sm < 1 ? 1 : per_sm));
            gather_rows_staged_kernel<<<(unsigned)blocks, STAGE_THREADS, smem, dl_cast(stream)>>>(x, map, out, B, F, M);
            return dl_launch_status();
        }
        cudaGetLastError();
    }
    const int64_t blocks = dl_min64(dl_ceil_div(B * M, 256), (int64_t)DL_NUM_SMS * 32);
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(x, map, out, B, F, M);
    return dl_launch_status();
}

DL_EXPORT int dl_gather_rows_bwd(const float* g, const int32_t* inv_ptr, const int32_t* inv_ent,
                                 float* gx, int64_t B, int64_t F, int64_t N, int64_t n,
                                 dl_stream_t stream) {
    DL_REQUIRE(g && inv_ptr && inv_ent && gx && B > 0 && F > 0 && N > 0 && n > 0);
    const int64_t M = N * n;
    const int64_t blocks = dl_min64(dl_ceil_div(dl_ceil_div(B, BWD_ROWS) * F, 256), (int64_t)DL_NUM_SMS * 32);
    gather_rows_bwd_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(g, inv_ptr, inv_ent, gx, B, F, M);
    return dl_launch_status();
}
