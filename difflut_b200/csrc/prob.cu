// Probabilistic node: multilinear expectation forward (optionally fused with GroupSum) and backward.
//
// out[b,v] = sum_a sigma(raw[v,a]/T) * prod_i (a_i ? x_i : 1 - x_i)  is the multilinear extension
// of the 2^n-entry table (difflut/nodes/probabilistic_node.py:263-300).  It is evaluated as an
// n-level interpolation tree (2^n - 1 lerps) instead of 2^n products of n factors; the backward is
// the same tree walked top-down, which yields d/dx_i and g*P_a(x) (the table gradient) together.
// Activations are feature-major fp32 [F][Bp]; the work is FP32-pipe bound, not HBM bound.
#include "common.cuh"

namespace {

constexpr int PROB_TILE = 128;  // samples per CTA in the forward kernel

// sigmoid(raw / max(T, 1e-6)) for one virtual node v = j*O + o, raw stored (N, L, O)
__device__ __forceinline__ float prob_weight(const float* __restrict__ raw, int64_t j, int o, int O,
                                             int L, int a, float inv_t) {
    const float z = __ldg(raw + (j * L + a) * O + o) * inv_t;
    return 1.0f / (1.0f + expf(-z));
}

// Interpolation tree on NIN inputs.  w[] holds 2^NIN weights; x[] the inputs.  Every loop has a
// compile-time trip count so that v[] stays in registers.
template <int NIN>
__device__ __forceinline__ float lerp_tree(const float* w, const float* x) {
    constexpr int H = 1 << (NIN > 0 ? NIN - 1 : 0);
    float v[H];
#pragma unroll
    for (int k = 0; k < H; ++k) v[k] = fmaf(x[0], w[2 * k + 1] - w[2 * k], w[2 * k]);
#pragma unroll
    for (int lvl = 1; lvl < NIN; ++lvl) {
#pragma unroll
        for (int k = 0; k < H / 2; ++k)
            if (k < (H >> lvl)) v[k] = fmaf(x[lvl], v[2 * k + 1] - v[2 * k], v[2 * k]);
    }
    return v[0];
}

// Forward.  CTA = (128-sample tile, slice of virtual nodes).  GROUPSUM: the slice lies inside one
// class and the CTA writes one partial sum row; otherwise every node writes its own output row.
template <int NIN, bool GROUPSUM>
__global__ void __launch_bounds__(PROB_TILE)
prob_fwd_kernel(const float* __restrict__ x_t, const int32_t* __restrict__ map,
                const float* __restrict__ raw, float inv_t, float* __restrict__ out_t,
                float* __restrict__ partial, int64_t NO, int O, int64_t gsz, int S, int64_t per,
                int64_t Bp) {
    constexpr int L = 1 << NIN;
    // two buffers: node v + 1 is staged while node v is evaluated, one barrier per node
    __shared__ float w_all[2][L];
    __shared__ int32_t rows_all[2][NIN];
    const int64_t b = (int64_t)blockIdx.x * PROB_TILE + threadIdx.x;
    int64_t v0, v1;
    if (GROUPSUM) {
        const int64_t cls = blockIdx.y / S, s = blockIdx.y % S;
        v0 = cls * gsz + s * per;
        v1 = v0 + per;
        if (v1 > (cls + 1) * gsz) v1 = (cls + 1) * gsz;
    } else {
        v0 = (int64_t)blockIdx.y * per;
        v1 = v0 + per;
    }
    if (v1 > NO) v1 = NO;
    float acc = 0.f;
    for (int64_t v = v0; v < v1; ++v) {
        const int64_t j = v / O;
        const int o = (int)(v - j * O);
        float* w = w_all[(v - v0) & 1];
        int32_t* rows = rows_all[(v - v0) & 1];
        if (threadIdx.x < L) w[threadIdx.x] = prob_weight(raw, j, o, O, L, threadIdx.x, inv_t);
        if (threadIdx.x < NIN) rows[threadIdx.x] = __ldg(map + j * NIN + threadIdx.x);
        // after this barrier the buffer is complete, and the other buffer (read for node v - 1) is free for v + 1
        __syncthreads();
        float x[NIN];
#pragma unroll
        for (int i = 0; i < NIN; ++i) x[i] = __ldg(x_t + (int64_t)rows[i] * Bp + b);
        const float y = lerp_tree<NIN>(w, x);
        if (GROUPSUM) acc += y;
        if (out_t != nullptr) out_t[v * Bp + b] = y;
    }
    if (GROUPSUM) partial[(int64_t)blockIdx.y * Bp + b] = acc;
}

__global__ void prob_groupsum_reduce_kernel(const float* __restrict__ partial, float* __restrict__ logits_t,
                                            int k, int S, float inv_tau, int64_t Bp) {
    const int64_t total = (int64_t)k * Bp;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = i / Bp, b = i - c * Bp;
        // eight loads in flight at a time; the additions keep their order, so the sum is unchanged
        const float* src = partial + c * S * Bp + b;
        float acc = 0.f;
        int s = 0;
        for (; s + 8 <= S; s += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldg(src + (int64_t)(s + u) * Bp);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += v[u];
        }
        for (; s < S; ++s) acc += __ldg(src + (int64_t)s * Bp);
        logits_t[i] = acc * inv_tau;
    }
}

// Backward.  One warp per node j; lane = sample, looping over the whole batch so the 2^n table gradient
// accumulators live in registers.  The inputs are split into a low group (NL inputs, address bits 0..NL-1)
// and a high group (NH inputs): P_a(x) = u[a_hi] * v[a_lo] with u, v the multilinear weights of each
// group (7 products each for 3 inputs).  Then
//   table gradient  acc[a_hi][a_lo] += (g u[a_hi]) * v[a_lo]                      (one FMA per entry)
//   s = W v, t = W^T u                                                           (two 2^n-FMA contractions)
//   d/dx_i for a high input = the derivative of the 2^NH-entry lerp tree over s, for a low input over t
// which is about 310 FP32 operations per (sample, node) for n = 6 and needs no per-sample array of 2^n
// entries besides the accumulators.  The node's table sits in shared memory (16-byte broadcast reads).
// gxm_t[(j*n+i)][b] receives the input gradient of slot i (summed over o).
// HYBRID (difflut/nodes/hybrid_node.py:173-224): `raw` holds the table values themselves in the DWN
// layout (N, O, 2^n), the table gradient is sum_b g*P_a with no sigmoid factor and is written in that
// layout, and d/dx_i carries the reference's factor x(1-x) / (x(1-x) + 1e-8), which makes the input
// gradient vanish at x in {0, 1}.

// out[k], k < 2^NB: product over the group's inputs of (bit i of k ? x[i] : 1 - x[i]), times `scale`
template <int NB>
__device__ __forceinline__ void group_weights(const float* x, float scale, float* out) {
    out[0] = scale;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
#pragma unroll
        for (int k = (1 << i) - 1; k >= 0; --k) {
            const float hi = out[k] * x[i];
            out[k + (1 << i)] = hi;
            out[k] = out[k] - hi;
        }
    }
}

// dx[i] = g * d/dx_i of the multilinear interpolation of tbl (2^NB entries) at x
template <int NB>
__device__ __forceinline__ void tree_gradient(const float* tbl, const float* x, float g, float* dx) {
    constexpr int L = 1 << NB;
    if (NB == 0) return;
    float d[L > 1 ? L - 1 : 1];
    float v[L > 1 ? L / 2 : 1];
#pragma unroll
    for (int k = 0; k < L / 2; ++k) {
        d[k] = tbl[2 * k + 1] - tbl[2 * k];
        v[k] = fmaf(x[0], d[k], tbl[2 * k]);
    }
#pragma unroll
    for (int lvl = 1; lvl < NB; ++lvl) {
        const int off = L - (L >> lvl);
#pragma unroll
        for (int k = 0; k < (L >> (lvl + 1)); ++k) {
            d[off + k] = v[2 * k + 1] - v[2 * k];
            v[k] = fmaf(x[lvl], d[off + k], v[2 * k]);
        }
    }
    float q[L > 1 ? L / 2 : 1];
    q[0] = g;
#pragma unroll
    for (int lvl = NB - 1; lvl >= 0; --lvl) {
        const int off = L - (L >> lvl);
        const int cnt = L >> (lvl + 1);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < cnt; ++k) acc = fmaf(q[k], d[off + k], acc);
        dx[lvl] = acc;
        if (lvl > 0) {
#pragma unroll
            for (int k = cnt - 1; k >= 0; --k) {
                const float hi = q[k] * x[lvl];
                q[2 * k + 1] = hi;
                q[2 * k] = q[k] - hi;
            }
        }
    }
}

template <int NIN, bool HYBRID>
__global__ void __launch_bounds__(128, 3)
prob_bwd_kernel(const float* __restrict__ x_t, const int32_t* __restrict__ map,
                const float* __restrict__ raw, float inv_t, const float* __restrict__ g_t,
                int64_t gdiv, float gscale, float* __restrict__ graw, float* __restrict__ gxm_t,
                int64_t N, int O, int64_t B, int64_t Bp) {
    constexpr int L = 1 << NIN;
    constexpr int NL = (NIN + 1) / 2, NH = NIN - NL;
    constexpr int LL = 1 << NL, LH = 1 << NH;
    __shared__ __align__(16) float w_all[4][L < 4 ? 4 : L];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* w = w_all[warp];
    const int64_t nwarps = (int64_t)gridDim.x * 4;
    for (int64_t j = (int64_t)blockIdx.x * 4 + warp; j < N; j += nwarps) {
        int32_t rows[NIN];
#pragma unroll
        for (int i = 0; i < NIN; ++i) rows[i] = __ldg(map + j * NIN + i);
        for (int o = 0; o < O; ++o) {
            __syncwarp();
            for (int a = lane; a < L; a += 32)
                w[a] = HYBRID ? __ldg(raw + (j * O + o) * L + a) : prob_weight(raw, j, o, O, L, a, inv_t);
            __syncwarp();
            float acc[L];
#pragma unroll
            for (int a = 0; a < L; ++a) acc[a] = 0.f;
            const float* grow = g_t + ((j * O + o) / gdiv) * Bp;
            for (int64_t b = lane; b < Bp; b += 32) {
                float x[NIN];
#pragma unroll
                for (int i = 0; i < NIN; ++i) x[i] = __ldg(x_t + (int64_t)rows[i] * Bp + b);
                const float g = (b < B) ? __ldg(grow + b) * gscale : 0.f;
                float u[LH], v[LL], gu[LH];
                group_weights<NL>(x, 1.f, v);
                group_weights<NH>(x + NL, 1.f, u);
#pragma unroll
                for (int h = 0; h < LH; ++h) gu[h] = g * u[h];
                // table gradient and the two contractions in one sweep over the table
                float s[LH], t[LL];
#pragma unroll
                for (int l = 0; l < LL; ++l) t[l] = 0.f;
#pragma unroll
                for (int h = 0; h < LH; ++h) {
                    float sh = 0.f;
#pragma unroll
                    for (int l = 0; l < LL; ++l) {
                        const float wv = w[h * LL + l];
                        acc[h * LL + l] = fmaf(gu[h], v[l], acc[h * LL + l]);
                        sh = fmaf(wv, v[l], sh);
                        t[l] = fmaf(wv, u[h], t[l]);
                    }
                    s[h] = sh;
                }
                if (gxm_t != nullptr) {
                    float dx[NIN];
                    tree_gradient<NL>(t, x, g, dx);
                    tree_gradient<NH>(s, x + NL, g, dx + NL);
#pragma unroll
                    for (int i = 0; i < NIN; ++i) {
                        float val = dx[i];
                        if (HYBRID) {
                            const float tt = x[i] * (1.f - x[i]);
                            val *= tt / (tt + 1e-8f);
                        }
                        float* dst = gxm_t + (j * NIN + i) * Bp + b;
                        if (o == 0) *dst = val; else *dst += val;
                    }
                }
            }
            // reduce the per-lane accumulators and apply sigma'(z)/T
            if (graw != nullptr) {
#pragma unroll
                for (int a = 0; a < L; ++a) {
                    float sum = acc[a];
#pragma unroll
                    for (int sh = 16; sh > 0; sh >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sh);
                    if (lane == (a & 31)) {
                        if (HYBRID) {
                            graw[(j * O + o) * L + a] = sum;
                        } else {
                            const float sg = w[a];
                            graw[(j * L + a) * O + o] = sum * sg * (1.f - sg) * inv_t;
                        }
                    }
                }
            }
        }
    }
}

// gx_t[f][b] = sum over CSR entries e of feature f of src_t[inv_ent[e]][b]
__global__ void seg_sum_t_kernel(const float* __restrict__ src_t, const int32_t* __restrict__ inv_ptr,
                                 const int32_t* __restrict__ inv_ent, float* __restrict__ gx_t,
                                 int64_t F, int64_t Bp) {
    const int64_t Q = Bp >> 2;
    const int64_t total = F * Q;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t f = t / Q, q = t - f * Q;
        const int e0 = __ldg(inv_ptr + f), e1 = __ldg(inv_ptr + f + 1);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int e = e0; e < e1; ++e) {
            const float4 s = __ldg(reinterpret_cast<const float4*>(src_t + (int64_t)__ldg(inv_ent + e) * Bp) + q);
            acc.x += s.x; acc.y += s.y; acc.z += s.z; acc.w += s.w;
        }
        reinterpret_cast<float4*>(gx_t + f * Bp)[q] = acc;
    }
}

template <bool GS>
int launch_fwd(int n, dim3 grid, cudaStream_t s, const float* x_t, const int32_t* map, const float* raw,
               float inv_t, float* out_t, float* partial, int64_t NO, int O, int64_t gsz, int S,
               int64_t per, int64_t Bp) {
    switch (n) {
        case 1: prob_fwd_kernel<1, GS><<<grid, PROB_TILE, 0, s>>>(x_t, map, raw, inv_t, out_t, partial, NO, O, gsz, S, per, Bp); break;
        case 2: prob_fwd_kernel<2, GS><<<grid, PROB_TILE, 0, s>>>(x_t, map, raw, inv_t, out_t, partial, NO, O, gsz, S, per, Bp); break;
        case 3: prob_fwd_kernel<3, GS><<<grid, PROB_TILE, 0, s>>>(x_t, map, raw, inv_t, out_t, partial, NO, O, gsz, S, per, Bp); break;
        case 4: prob_fwd_kernel<4, GS><<<grid, PROB_TILE, 0, s>>>(x_t, map, raw, inv_t, out_t, partial, NO, O, gsz, S, per, Bp); break;
        case 5: prob_fwd_kernel<5, GS><<<grid, PROB_TILE, 0, s>>>(x_t, map, raw, inv_t, out_t, partial, NO, O, gsz, S, per, Bp); break;
        case 6: prob_fwd_kernel<6, GS><<<grid, PROB_TILE, 0, s>>>(x_t, map, raw, inv_t, out_t, partial, NO, O, gsz, S, per, Bp); break;
        default: return DL_ERR_UNSUPPORTED;
    }
    return dl_launch_status();
}

}  // namespace

DL_EXPORT int dl_prob_fwd_t(const float* x_t, const int32_t* map, const float* raw, float temperature,
                            float* out_t, int64_t N, int64_t n, int64_t O, int64_t Bp,
                            dl_stream_t stream) {
    DL_REQUIRE(x_t && map && raw && out_t && N > 0 && O > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const float inv_t = 1.0f / fmaxf(temperature, 1e-6f);
    const int64_t NO = N * O;
    // slices sized so the grid has a few CTAs per SM
    const int64_t tiles = Bp / PROB_TILE;
    int64_t slices = dl_ceil_div((int64_t)DL_NUM_SMS * 8, tiles);
    if (slices > NO) slices = NO;
    if (slices > 65535) slices = 65535;
    const int64_t per = dl_ceil_div(NO, slices);
    slices = dl_ceil_div(NO, per);
    dim3 grid((unsigned)tiles, (unsigned)slices);
    return launch_fwd<false>((int)n, grid, dl_cast(stream), x_t, map, raw, inv_t, out_t, nullptr, NO, (int)O, 0,
                             1, per, Bp);
}

DL_EXPORT int64_t dl_prob_groupsum_splits(int64_t NO, int64_t k) {
    if (NO <= 0 || k <= 0) return 1;
    const int64_t gsz = dl_ceil_div(NO, k);
    int64_t s = gsz / 16;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return s;
}

DL_EXPORT int dl_prob_fwd_groupsum_t(const float* x_t, const int32_t* map, const float* raw,
                                     float temperature, float* out_t, float* partial, float* logits_t,
                                     int64_t N, int64_t n, int64_t O, int64_t k, float tau, int64_t Bp,
                                     dl_stream_t stream) {
    DL_REQUIRE(x_t && map && raw && partial && logits_t && N > 0 && O > 0 && k > 0 && tau > 0.f);
    DL_REQUIRE(Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const float inv_t = 1.0f / fmaxf(temperature, 1e-6f);
    const int64_t NO = N * O;
    const int64_t gsz = dl_ceil_div(NO, k);
    const int S = (int)dl_prob_groupsum_splits(NO, k);
    const int64_t per = dl_ceil_div(gsz, S);
    DL_REQUIRE(k * S <= 65535);
    dim3 grid((unsigned)(Bp / PROB_TILE), (unsigned)(k * S));
    const int rc = launch_fwd<true>((int)n, grid, dl_cast(stream), x_t, map, raw, inv_t, out_t, partial, NO,
                                    (int)O, gsz, S, per, Bp);
    if (rc != DL_OK) return rc;
    const int64_t blocks = dl_min64(dl_ceil_div(k * Bp, 256), (int64_t)DL_NUM_SMS * 8);
    prob_groupsum_reduce_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(partial, logits_t, (int)k, S,
                                                                             1.0f / tau, Bp);
    return dl_launch_status();
}

template <bool HYBRID>
static int launch_prob_bwd(const float* x_t, const int32_t* map, const float* raw, float inv_t, const float* g_t,
                           int64_t gdiv, float gscale, float* graw, float* gxm_t, int64_t N, int64_t n, int64_t O,
                           int64_t B, int64_t Bp, cudaStream_t s) {
    const int64_t blocks = dl_min64(dl_ceil_div(N, 4), (int64_t)DL_NUM_SMS * 16);
    const unsigned gb = (unsigned)blocks;
    switch (n) {
        case 1: prob_bwd_kernel<1, HYBRID><<<gb, 128, 0, s>>>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, (int)O, B, Bp); break;
        case 2: prob_bwd_kernel<2, HYBRID><<<gb, 128, 0, s>>>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, (int)O, B, Bp); break;
        case 3: prob_bwd_kernel<3, HYBRID><<<gb, 128, 0, s>>>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, (int)O, B, Bp); break;
        case 4: prob_bwd_kernel<4, HYBRID><<<gb, 128, 0, s>>>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, (int)O, B, Bp); break;
        case 5: prob_bwd_kernel<5, HYBRID><<<gb, 128, 0, s>>>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, (int)O, B, Bp); break;
        default: prob_bwd_kernel<6, HYBRID><<<gb, 128, 0, s>>>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, (int)O, B, Bp); break;
    }
    return dl_launch_status();
}

DL_EXPORT int dl_prob_bwd_t(const float* x_t, const int32_t* map, const float* raw, float temperature,
                            const float* g_t, int64_t gdiv, float gscale, float* graw, float* gxm_t,
                            int64_t N, int64_t n, int64_t O, int64_t B, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(x_t && map && raw && g_t && (graw || gxm_t) && N > 0 && O > 0 && gdiv > 0);
    DL_REQUIRE(B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const float inv_t = 1.0f / fmaxf(temperature, 1e-6f);
    return launch_prob_bwd<false>(x_t, map, raw, inv_t, g_t, gdiv, gscale, graw, gxm_t, N, n, O, B, Bp,
                                  dl_cast(stream));
}

DL_EXPORT int dl_hybrid_bwd_t(const float* x_t, const int32_t* map, const float* tables, const float* g_t,
                              int64_t gdiv, float gscale, float* gtables, float* gxm_t, int64_t N, int64_t n,
                              int64_t O, int64_t B, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(x_t && map && tables && g_t && (gtables || gxm_t) && N > 0 && O > 0 && gdiv > 0);
    DL_REQUIRE(B > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    return launch_prob_bwd<true>(x_t, map, tables, 1.0f, g_t, gdiv, gscale, gtables, gxm_t, N, n, O, B, Bp,
                                 dl_cast(stream));
}

DL_EXPORT int dl_seg_sum_t(const float* src_t, const int32_t* inv_ptr, const int32_t* inv_ent, float* gx_t,
                           int64_t F, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(src_t && inv_ptr && inv_ent && gx_t && F > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(src_t, 16);
    DL_REQUIRE_ALIGNED(gx_t, 16);
    const int64_t blocks = dl_min64(dl_ceil_div(F * (Bp / 4), 256), (int64_t)DL_NUM_SMS * 16);
    seg_sum_t_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(src_t, inv_ptr, inv_ent, gx_t, F, Bp);
    return dl_launch_status();
}
