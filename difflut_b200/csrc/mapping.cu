// RandomLayer gather on fp32 rows and its scatter-add backward (API-exact `get_mapping`).
//
// Forward is a plain indexed copy.  The backward replaces the reference's global fp32 atomics
// (difflut/layers/cuda/mapping_cuda_kernel.cu:136-162) by a segmented sum over the inverse map:
// thread (b, f) adds the gradient columns listed for feature f in a fixed order.
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

__global__ void gather_rows_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ inv_ptr,
                                       const int32_t* __restrict__ inv_ent, float* __restrict__ gx,
                                       int64_t B, int64_t F, int64_t M) {
    const int64_t total = B * F;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = t / F, f = t - b * F;
        const int e0 = __ldg(inv_ptr + f), e1 = __ldg(inv_ptr + f + 1);
        float acc = 0.f;
        for (int e = e0; e < e1; ++e) acc += __ldg(g + b * M + __ldg(inv_ent + e));
        gx[t] = acc;
    }
}

}  // namespace

DL_EXPORT int dl_gather_rows(const float* x, const int32_t* map, float* out, int64_t B, int64_t F,
                             int64_t N, int64_t n, dl_stream_t stream) {
    DL_REQUIRE(x && map && out && B > 0 && F > 0 && N > 0 && n > 0);
    const int64_t blocks = dl_min64(dl_ceil_div(B * N * n, 256), (int64_t)DL_NUM_SMS * 32);
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(x, map, out, B, F, N * n);
    return dl_launch_status();
}

DL_EXPORT int dl_gather_rows_bwd(const float* g, const int32_t* inv_ptr, const int32_t* inv_ent,
                                 float* gx, int64_t B, int64_t F, int64_t N, int64_t n,
                                 dl_stream_t stream) {
    DL_REQUIRE(g && inv_ptr && inv_ent && gx && B > 0 && F > 0 && N > 0 && n > 0);
    const int64_t blocks = dl_min64(dl_ceil_div(B * F, 256), (int64_t)DL_NUM_SMS * 32);
    gather_rows_bwd_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(g, inv_ptr, inv_ent, gx, B, F,
                                                                        N * n);
    return dl_launch_status();
}
