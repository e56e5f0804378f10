// DWNStable and Hybrid node backward for 6 < n <= 16 inputs per node, on materialised inputs xm (B, N, n).
//
// The n <= 6 layer kernels keep a node's whole backward transform in 32 lanes (dwn.cu) or its 2^n table
// gradient in registers (prob.cu); neither fits here.  These kernels restate the reference's per-sample
// sums directly, one thread per output element, tables read from global memory: they exist so that every
// node size the reference accepts runs on the GPU, not to be fast.
//   DWNStable  difflut/nodes/dwn_stable_node.py:145-205
//   Hybrid     difflut/nodes/hybrid_node.py:160-224
#include "common.cuh"

namespace {

constexpr int WIDE_MAX_N = 16;

__device__ __forceinline__ int wide_addr(const float* __restrict__ x, int n) {
    int a = 0;
    for (int i = 0; i < n; ++i) a |= (x[i] >= 0.5f ? 1 : 0) << i;
    return a;
}

// thread per (b, j, i): gxm[b,j,i] = scale_j * sum_o g[b,j,o] * sum_k sgn(k_i) lut[j,o,k] / (hamming + 1),
// hamming = popcount((addr ^ k) without bit i).  Accumulated in double: the slowly decaying weights leave a
// heavily cancelling sum (the reference accumulates in Python floats).
__global__ void stable_wide_bwd_input_kernel(const float* __restrict__ xm, const float* __restrict__ tables,
                                             const float* __restrict__ g, const float* __restrict__ scale_node,
                                             float scale, float* __restrict__ gxm, int64_t B, int64_t N, int n,
                                             int O) {
    const int L = 1 << n;
    const int64_t total = B * N * n;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)(t % n);
        const int64_t bj = t / n, j = bj % N;
        const int a = wide_addr(xm + bj * n, n);
        const int keep = (L - 1) & ~(1 << i);
        double total_grad = 0.0;
        for (int o = 0; o < O; ++o) {
            const float* lut = tables + (j * O + o) * (int64_t)L;
            double acc = 0.0;
            for (int k = 0; k < L; ++k) {
                const double term = (double)__ldg(lut + k) / (double)(__popc((a ^ k) & keep) + 1);
                acc += ((k >> i) & 1) ? term : -term;
            }
            total_grad += acc * (double)g[bj * O + o];
        }
        const double s = scale_node != nullptr ? (double)scale_node[j] : (double)scale;
        gxm[t] = (float)(s * total_grad);
    }
}

// thread per (b, j): P[a] = prod_i (a_i ? x_i : 1 - x_i); table gradient by fp32 atomics (gt zeroed by the entry
// point), input gradient in double throughout: with tables that vary little the 2^n signed terms of an input
// gradient cancel almost completely, and the rounding of fp32 terms would show at the 1e-5 level.
__global__ void hybrid_wide_bwd_kernel(const float* __restrict__ xm, const float* __restrict__ tables,
                                       const float* __restrict__ g, float* __restrict__ gxm, float* __restrict__ gt,
                                       int64_t B, int64_t N, int n, int O) {
    const int L = 1 << n;
    const int64_t total = B * N;
    for (int64_t bj = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; bj < total;
         bj += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = bj % N;
        double x[WIDE_MAX_N], inv[WIDE_MAX_N], gx[WIDE_MAX_N];
        for (int i = 0; i < WIDE_MAX_N; ++i) {
            x[i] = i < n ? (double)xm[bj * n + i] : 0.0;
            inv[i] = 1.0 / (x[i] * (1.0 - x[i]) + 1e-8);
            gx[i] = 0.0;
        }
        for (int a = 0; a < L; ++a) {
            double p = 1.0;
            for (int i = 0; i < n; ++i) p *= ((a >> i) & 1) ? x[i] : 1.0 - x[i];
            double lg = 0.0;  // sum_o table[j,o,a] * g[b,j,o]
            for (int o = 0; o < O; ++o) {
                const float go = g[bj * O + o];
                lg += (double)__ldg(tables + (j * O + o) * (int64_t)L + a) * (double)go;
                if (gt != nullptr && p != 0.0) atomicAdd(gt + (j * O + o) * (int64_t)L + a, (float)(p * (double)go));
            }
            if (gxm != nullptr && p != 0.0 && lg != 0.0)
                for (int i = 0; i < n; ++i) gx[i] += p * ((((a >> i) & 1) ? 1.0 : 0.0) - x[i]) * inv[i] * lg;
        }
        if (gxm != nullptr)
            for (int i = 0; i < n; ++i) gxm[bj * n + i] = (float)gx[i];
    }
}

int wide_grid(int64_t threads) {
    const int64_t blocks = dl_ceil_div(threads, 128);
    const int64_t cap = (int64_t)DL_NUM_SMS * 32;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace

DL_EXPORT int dl_dwn_stable_mapped_bwd_input(const float* xm, const float* tables, const float* g,
                                             const float* scale_per_node, float scale, float* gxm, int64_t B,
                                             int64_t N, int64_t n, int64_t O, dl_stream_t stream) {
    DL_REQUIRE(xm && tables && g && gxm && B > 0 && N > 0 && O > 0);
    if (n < 1 || n > WIDE_MAX_N) return DL_ERR_UNSUPPORTED;
    stable_wide_bwd_input_kernel<<<wide_grid(B * N * n), 128, 0, dl_cast(stream)>>>(xm, tables, g, scale_per_node, scale,
                                                                                gxm, B, N, (int)n, (int)O);
    return dl_launch_status();
}

DL_EXPORT int dl_hybrid_mapped_bwd(const float* xm, const float* tables, const float* g, float* gxm, float* gt,
                                   int64_t B, int64_t N, int64_t n, int64_t O, dl_stream_t stream) {
    DL_REQUIRE(xm && tables && g && (gxm || gt) && B > 0 && N > 0 && O > 0);
    if (n < 1 || n > WIDE_MAX_N) return DL_ERR_UNSUPPORTED;
    cudaStream_t s = dl_cast(stream);
    if (gt != nullptr && cudaMemsetAsync(gt, 0, sizeof(float) * N * O * ((int64_t)1 << n), s) != cudaSuccess)
        return DL_ERR_LAUNCH;
    hybrid_wide_bwd_kernel<<<wide_grid(B * N), 128, 0, s>>>(xm, tables, g, gxm, gt, B, N, (int)n, (int)O);
    return dl_launch_status();
}
