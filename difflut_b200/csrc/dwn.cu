// DWN node kernels: LUT forward, extended-finite-difference (EFD) backward.
//
// Feature-major path ("_t"): activations are bit-packed [F][Bp/32]; a warp works on one node
// (or one input feature) and its lanes on consecutive samples, so every global access is a
// coalesced row segment.  Per sample the EFD backward is one address, one histogram update and
// n lookups in the per-step transform table `efd_t` instead of the reference's 2^n-term loop
// (difflut/nodes/dwn_node.py:195-227).
#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------
// per-step table preparation
// ------------------------------------------------------------------------------------------

// One CTA per node (grid-stride).  Threads (i, a') with i < n, a' < 2^(n-1) evaluate the
// reference's inner sum over k directly, in double, with sign and beta^hamming weights.
__global__ void __launch_bounds__(192)
dwn_prepare_kernel(const float* __restrict__ tables, float* __restrict__ efd_t,
                   uint64_t* __restrict__ masks, int64_t N, int n, float alpha, float beta) {
    __shared__ float lut[64];
    __shared__ double bpow[8];
    const int L = 1 << n;
    if (threadIdx.x < 8) bpow[threadIdx.x] = pow((double)beta, (double)threadIdx.x);
    for (int64_t j = blockIdx.x; j < N; j += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < L) lut[threadIdx.x] = tables[j * L + threadIdx.x];
        __syncthreads();
        if (masks != nullptr && threadIdx.x < 32) {
            const int lane = threadIdx.x;
            const uint32_t lo = __ballot_sync(0xffffffffu, lane < L && lut[lane] >= 0.5f);
            const uint32_t hi = __ballot_sync(0xffffffffu, lane + 32 < L && lut[(lane + 32) & 63] >= 0.5f);
            if (lane == 0) masks[j] = ((uint64_t)hi << 32) | lo;
        }
        if (efd_t != nullptr) {
            const int i = threadIdx.x >> 5, a5 = threadIdx.x & 31;
            if (i < n) {
                double acc = 0.0;
                if (a5 < (L >> 1)) {
                    const int low = (1 << i) - 1;
                    const int a = ((a5 & ~low) << 1) | (a5 & low);  // bit i of a is 0
                    const int keep = (L - 1) & ~(1 << i);
                    for (int k = 0; k < L; ++k) {
                        const int ham = __popc((a ^ k) & keep);
                        const double term = (double)lut[k] * bpow[ham];
                        acc += ((k >> i) & 1) ? term : -term;
                    }
                }
                efd_t[(j * n + i) * 32 + a5] = (float)((double)alpha * acc);
            }
        }
    }
}

// General n: separable butterfly.  One CTA per (virtual node v, input slot i); the slab
// efd_full[v][i][0..L) starts as a copy of the table and is transformed in place along every
// address bit: bit i -> (v1 - v0) in both halves, other bits -> (v0 + beta v1, beta v0 + v1).
__global__ void __launch_bounds__(256)
dwn_prepare_full_kernel(const float* __restrict__ tables, float* __restrict__ efd_full, int64_t NO,
                        int n, float alpha, float beta) {
    const int L = 1 << n;
    for (int64_t item = blockIdx.x; item < NO * n; item += gridDim.x) {
        const int64_t v = item / n;
        const int i = (int)(item % n);
        float* slab = efd_full + item * L;
        for (int a = threadIdx.x; a < L; a += blockDim.x) slab[a] = alpha * tables[v * L + a];
        __syncthreads();
        for (int bit = 0; bit < n; ++bit) {
            const int stride = 1 << bit;
            for (int p = threadIdx.x; p < (L >> 1); p += blockDim.x) {
                const int lo = ((p >> bit) << (bit + 1)) | (p & (stride - 1));
                const int hi = lo | stride;
                const float v0 = slab[lo], v1 = slab[hi];
                if (bit == i) {
                    slab[lo] = v1 - v0;
                    slab[hi] = v1 - v0;
                } else {
                    slab[lo] = v0 + beta * v1;
                    slab[hi] = beta * v0 + v1;
                }
            }
            __syncthreads();
        }
    }
}

// ------------------------------------------------------------------------------------------
// bit-sliced hard forward
// ------------------------------------------------------------------------------------------

// Depth-first evaluation of the 2^n -> 1 multiplexer tree on 4 words (128 samples) at once.
// A leaf turns two adjacent truth-table bits into all-zero / all-one masks and selects with
// input 0; every inner node is one select on input LVL.  BASE and LVL are compile-time, so
// every shift is an immediate and the tree is 2^n - 1 three-input logic ops per word.
template <int LVL, int BASE>
struct MuxTree {
    __device__ __forceinline__ static void eval(uint32_t lo, uint32_t hi, const uint4* x, uint4& out) {
        uint4 a, b;
        MuxTree<LVL - 1, BASE>::eval(lo, hi, x, a);
        MuxTree<LVL - 1, BASE + (1 << LVL)>::eval(lo, hi, x, b);
        const uint4 s = x[LVL];
        out.x = (a.x & ~s.x) | (b.x & s.x);
        out.y = (a.y & ~s.y) | (b.y & s.y);
        out.z = (a.z & ~s.z) | (b.z & s.z);
        out.w = (a.w & ~s.w) | (b.w & s.w);
    }
};
template <int BASE>
struct MuxTree<0, BASE> {
    __device__ __forceinline__ static void eval(uint32_t lo, uint32_t hi, const uint4* x, uint4& out) {
        const uint32_t word = BASE < 32 ? lo : hi;
        const uint32_t c0 = 0u - ((word >> (BASE & 31)) & 1u);
        const uint32_t c1 = 0u - ((word >> ((BASE + 1) & 31)) & 1u);
        const uint4 s = x[0];
        out.x = (c0 & ~s.x) | (c1 & s.x);
        out.y = (c0 & ~s.y) | (c1 & s.y);
        out.z = (c0 & ~s.z) | (c1 & s.z);
        out.w = (c0 & ~s.w) | (c1 & s.w);
    }
};

// Work item = (node j, group of 4 words).  Q = Wp/4 groups per node; items are numbered with the
// word group fastest so a warp reads contiguous 512-byte segments of each input row.
template <int NIN>
__global__ void __launch_bounds__(256)
dwn_fwd_bits_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                    const uint64_t* __restrict__ masks, uint32_t* __restrict__ out_bits, int64_t N,
                    int64_t Wp) {
    const int64_t Q = Wp >> 2;
    const int64_t total = N * Q;
    for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < total;
         item += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = item / Q, q = item - j * Q;
        const uint64_t m = __ldg(&masks[j]);
        uint4 x[NIN];
#pragma unroll
        for (int i = 0; i < NIN; ++i) {
            const int64_t row = __ldg(&map[j * NIN + i]);
            x[i] = __ldg(reinterpret_cast<const uint4*>(in_bits + row * Wp) + q);
        }
        uint4 o;
        MuxTree<NIN - 1, 0>::eval((uint32_t)m, (uint32_t)(m >> 32), x, o);
        reinterpret_cast<uint4*>(out_bits + j * Wp)[q] = o;
    }
}

// ------------------------------------------------------------------------------------------
// per-sample addresses
// ------------------------------------------------------------------------------------------

// Addresses of 4 consecutive samples (b0 multiple of 4) of one node, one per byte.
__device__ __forceinline__ uint32_t addr4(const uint32_t* __restrict__ in_bits, const int32_t* rows,
                                          int n, int64_t Wp, int64_t b0) {
    const int64_t word = b0 >> 5;
    const int sh = (int)(b0 & 31);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < DL_MAX_FAST_N; ++i) {
        if (i < n) {
            const uint32_t w = __ldg(in_bits + (int64_t)rows[i] * Wp + word);
            packed |= dl_spread_nibble((w >> sh) & 0xFu) << i;
        }
    }
    return packed;
}

// Training forward, one warp per (node, 128-sample chunk); lane = 4 consecutive samples.
__global__ void __launch_bounds__(256)
dwn_fwd_vals_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                    const float* __restrict__ tables, float* __restrict__ out_t,
                    uint8_t* __restrict__ addr_t, int64_t N, int n, int64_t Bp) {
    const int lane = threadIdx.x & 31;
    const int64_t C = Bp >> 7, Wp = Bp >> 5;
    const int L = 1 << n;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < N * C;
         item += nwarps) {
        const int64_t j = item / C, c = item - j * C;
        int32_t rows[DL_MAX_FAST_N];
#pragma unroll
        for (int i = 0; i < DL_MAX_FAST_N; ++i) rows[i] = i < n ? __ldg(&map[j * n + i]) : 0;
        const int64_t b = (c << 7) + lane * 4;
        const uint32_t a = addr4(in_bits, rows, n, Wp, b);
        const float* tj = tables + j * L;
        float4 o;
        o.x = __ldg(tj + (a & 0xFF));
        o.y = __ldg(tj + ((a >> 8) & 0xFF));
        o.z = __ldg(tj + ((a >> 16) & 0xFF));
        o.w = __ldg(tj + (a >> 24));
        *reinterpret_cast<float4*>(out_t + j * Bp + b) = o;
        if (addr_t != nullptr) *reinterpret_cast<uint32_t*>(addr_t + j * Bp + b) = a;
    }
}

// Last layer fused with GroupSum: CTA (x = 512-sample tile, y = class*S + slice); each warp
// walks the nodes of its slice and keeps 4 running sums per lane.
__global__ void __launch_bounds__(128)
dwn_fwd_groupsum_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                        const float* __restrict__ tables, float* __restrict__ partial, int64_t N,
                        int n, int64_t gsz, int S, int64_t Bp) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t Wp = Bp >> 5;
    const int L = 1 << n;
    const int64_t b = ((int64_t)blockIdx.x * 4 + warp) * 128 + lane * 4;
    if (b >= Bp) return;
    const int64_t cls = blockIdx.y / S, s = blockIdx.y % S;
    const int64_t per = dl_ceil_div_dev(gsz, S);
    const int64_t j0 = cls * gsz + s * per;
    int64_t j1 = j0 + per;
    if (j1 > (cls + 1) * gsz) j1 = (cls + 1) * gsz;
    if (j1 > N) j1 = N;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t j = j0; j < j1; ++j) {
        int32_t rows[DL_MAX_FAST_N];
#pragma unroll
        for (int i = 0; i < DL_MAX_FAST_N; ++i) rows[i] = i < n ? __ldg(&map[j * n + i]) : 0;
        const uint32_t a = addr4(in_bits, rows, n, Wp, b);
        const float* tj = tables + j * L;
        acc.x += __ldg(tj + (a & 0xFF));
        acc.y += __ldg(tj + ((a >> 8) & 0xFF));
        acc.z += __ldg(tj + ((a >> 16) & 0xFF));
        acc.w += __ldg(tj + (a >> 24));
    }
    *reinterpret_cast<float4*>(partial + (int64_t)blockIdx.y * Bp + b) = acc;
}

__global__ void groupsum_reduce_kernel(const float* __restrict__ partial, float* __restrict__ logits_t,
                                       int k, int S, float inv_tau, int64_t Bp) {
    const int64_t total = (int64_t)k * Bp;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = i / Bp, b = i - c * Bp;
        float acc = 0.f;
        for (int s = 0; s < S; ++s) acc += partial[(c * S + s) * Bp + b];
        logits_t[i] = acc * inv_tau;
    }
}

// ------------------------------------------------------------------------------------------
// backward: table gradient (histogram) and input gradient (segmented pull)
// ------------------------------------------------------------------------------------------

constexpr int HIST_WARPS = 4;

// One warp per node.  hist[e][lane] is private to the lane (bank = lane: conflict-free, no
// atomics); the chunk loop adds each sample's gradient to the bin of its address, then the 32
// lane copies of each bin are summed in a rotated order (again conflict-free).
__global__ void __launch_bounds__(HIST_WARPS * 32)
dwn_bwd_tables_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                      const float* __restrict__ g_t, int64_t gdiv, float gscale,
                      float* __restrict__ gt, uint8_t* __restrict__ addr_t, int64_t N, int n,
                      int64_t Bp) {
    __shared__ float hist_all[HIST_WARPS][64][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float(*hist)[32] = hist_all[warp];
    const int64_t C = Bp >> 7, Wp = Bp >> 5;
    const int L = 1 << n;
    const int64_t nwarps = (int64_t)gridDim.x * HIST_WARPS;
    for (int64_t j = (int64_t)blockIdx.x * HIST_WARPS + warp; j < N; j += nwarps) {
        int32_t rows[DL_MAX_FAST_N];
#pragma unroll
        for (int i = 0; i < DL_MAX_FAST_N; ++i) rows[i] = i < n ? __ldg(&map[j * n + i]) : 0;
#pragma unroll 8
        for (int e = 0; e < 64; ++e) hist[e][lane] = 0.f;
        const float* grow = g_t + (j / gdiv) * Bp;
        for (int64_t c = 0; c < C; ++c) {
            const int64_t b = (c << 7) + lane * 4;
            const uint32_t a = addr4(in_bits, rows, n, Wp, b);
            const float4 g = __ldg(reinterpret_cast<const float4*>(grow + b));
            if (addr_t != nullptr) *reinterpret_cast<uint32_t*>(addr_t + j * Bp + b) = a;
            hist[a & 0xFF][lane] += g.x * gscale;
            hist[(a >> 8) & 0xFF][lane] += g.y * gscale;
            hist[(a >> 16) & 0xFF][lane] += g.z * gscale;
            hist[a >> 24][lane] += g.w * gscale;
        }
        __syncwarp();
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
        for (int r = 0; r < 32; ++r) {
            const int col = (r + lane) & 31;
            s0 += hist[lane][col];
            s1 += hist[lane + 32][col];
        }
        if (lane < L) gt[j * L + lane] = s0;
        if (lane + 32 < L) gt[j * L + lane + 32] = s1;
        __syncwarp();
    }
}

// One warp per (input feature f, 128-sample chunk).  For every (node j, slot i) that reads f the
// 32 distinct EFD values of (j,i) sit one per lane and each sample fetches its value with a
// single shuffle indexed by its address without bit i.
__global__ void __launch_bounds__(256)
dwn_bwd_input_kernel(const uint8_t* __restrict__ addr_t, const float* __restrict__ g_t, int64_t gdiv,
                     float gscale, const float* __restrict__ efd_t,
                     const int32_t* __restrict__ inv_ptr, const int32_t* __restrict__ inv_ent,
                     float* __restrict__ gx_t, int64_t F, int n, int64_t Bp) {
    const int lane = threadIdx.x & 31;
    const int64_t C = Bp >> 7;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < F * C;
         item += nwarps) {
        const int64_t f = item / C, c = item - f * C;
        const int64_t b = (c << 7) + lane * 4;
        const int e0 = __ldg(&inv_ptr[f]), e1 = __ldg(&inv_ptr[f + 1]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int e = e0; e < e1; ++e) {
            const int ent = __ldg(&inv_ent[e]);
            const int j = ent / n, i = ent - j * n;
            const float tv = __ldg(efd_t + (int64_t)ent * 32 + lane);
            const uint32_t a = __ldg(reinterpret_cast<const uint32_t*>(addr_t + (int64_t)j * Bp + b));
            const float4 g = __ldg(reinterpret_cast<const float4*>(g_t + (int64_t)(j / gdiv) * Bp + b));
            const uint32_t low = (1u << i) - 1u;
            // drop bit i of every byte: keep the bits below i, shift the bits above i down by one
            const uint32_t lowm = low * 0x01010101u;
            const uint32_t a5 = (a & lowm) | ((a >> 1) & ~lowm & 0x7F7F7F7Fu);
            acc.x += g.x * __shfl_sync(0xffffffffu, tv, a5 & 31);
            acc.y += g.y * __shfl_sync(0xffffffffu, tv, (a5 >> 8) & 31);
            acc.z += g.z * __shfl_sync(0xffffffffu, tv, (a5 >> 16) & 31);
            acc.w += g.w * __shfl_sync(0xffffffffu, tv, (a5 >> 24) & 31);
        }
        acc.x *= gscale; acc.y *= gscale; acc.z *= gscale; acc.w *= gscale;
        *reinterpret_cast<float4*>(gx_t + f * Bp + b) = acc;
    }
}

// ------------------------------------------------------------------------------------------
// materialised-input path: xm (B, N, n) rows
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ int mapped_addr(const float* __restrict__ x, int n, int L, bool eval_mode) {
    if (!eval_mode) {
        int a = 0;
        for (int i = 0; i < n; ++i) a |= (x[i] >= 0.5f ? 1 : 0) << i;
        return a;
    }
    // eval: the reference forms the index in float arithmetic from inputs that are already {0,1}
    // (difflut/nodes/dwn_node.py:469-473); out-of-range results are clamped instead of faulting
    float s = 0.f;
    for (int i = 0; i < n; ++i) s += x[i] * (float)(1 << i);
    int a = (int)s;
    return a < 0 ? 0 : (a >= L ? L - 1 : a);
}

__global__ void dwn_mapped_fwd_kernel(const float* __restrict__ xm, const float* __restrict__ tables,
                                      float* __restrict__ out, int64_t B, int64_t N, int n, int O,
                                      bool eval_mode) {
    const int L = 1 << n;
    const int64_t total = B * N;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = t % N;
        const int a = mapped_addr(xm + t * n, n, L, eval_mode);
        for (int o = 0; o < O; ++o) {
            const float v = __ldg(tables + (j * O + o) * L + a);
            out[t * O + o] = eval_mode ? (v >= 0.5f ? 1.f : 0.f) : v;
        }
    }
}

__global__ void dwn_mapped_bwd_input_kernel(const float* __restrict__ xm, const float* __restrict__ g,
                                            const float* __restrict__ efd_full,
                                            float* __restrict__ gxm, int64_t B, int64_t N, int n,
                                            int O) {
    const int L = 1 << n;
    const int64_t total = B * N;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = t % N;
        const int a = mapped_addr(xm + t * n, n, L, false);
        for (int i = 0; i < n; ++i) {
            float acc = 0.f;
            for (int o = 0; o < O; ++o)
                acc += g[t * O + o] * __ldg(efd_full + ((j * O + o) * n + i) * (int64_t)L + a);
            gxm[t * n + i] = acc;
        }
    }
}

// n <= 6: CTA owns 32 consecutive virtual nodes v = j*O + o (lane = v), warps stride over the
// batch; lane-private histograms as above, then the HIST_WARPS copies are added in order.
__global__ void __launch_bounds__(HIST_WARPS * 32)
dwn_mapped_bwd_tables_kernel(const float* __restrict__ xm, const float* __restrict__ g,
                             float* __restrict__ gt, int64_t B, int64_t N, int n, int O) {
    __shared__ float hist[HIST_WARPS][64][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int L = 1 << n;
    const int64_t NO = N * O;
    const int64_t v = (int64_t)blockIdx.x * 32 + lane;
    for (int e = 0; e < 64; ++e) hist[warp][e][lane] = 0.f;
    if (v < NO) {
        const int64_t j = v / O;
        for (int64_t b = warp; b < B; b += HIST_WARPS) {
            const int a = mapped_addr(xm + (b * N + j) * n, n, L, false);
            hist[warp][a][lane] += g[b * NO + v];
        }
    }
    __syncthreads();
    if (v < NO) {
        for (int e = warp; e < L; e += HIST_WARPS) {
            float s = 0.f;
            for (int w = 0; w < HIST_WARPS; ++w) s += hist[w][e][lane];
            gt[v * L + e] = s;
        }
    }
}

// n > 6: gt is zeroed by the caller-side memset below, then fp32 atomics.
__global__ void dwn_mapped_bwd_tables_atomic_kernel(const float* __restrict__ xm,
                                                    const float* __restrict__ g,
                                                    float* __restrict__ gt, int64_t B, int64_t N,
                                                    int n, int O) {
    const int L = 1 << n;
    const int64_t total = B * N;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = t % N;
        const int a = mapped_addr(xm + t * n, n, L, false);
        for (int o = 0; o < O; ++o) atomicAdd(gt + (j * O + o) * (int64_t)L + a, g[t * O + o]);
    }
}

int grid_for(int64_t threads_needed, int block) {
    const int64_t blocks = dl_ceil_div(threads_needed, block);
    const int64_t cap = (int64_t)DL_NUM_SMS * 32;
    return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

DL_EXPORT int dl_dwn_prepare(const float* tables, float* efd_t, uint64_t* masks, int64_t N, int64_t n,
                             float alpha, float beta, dl_stream_t stream) {
    DL_REQUIRE(tables && N > 0 && (efd_t || masks));
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int blocks = (int)(N < (int64_t)DL_NUM_SMS * 16 ? N : (int64_t)DL_NUM_SMS * 16);
    dwn_prepare_kernel<<<blocks, 192, 0, dl_cast(stream)>>>(tables, efd_t, masks, N, (int)n, alpha, beta);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_prepare_full(const float* tables, float* efd_full, int64_t NO, int64_t n,
                                  float alpha, float beta, dl_stream_t stream) {
    DL_REQUIRE(tables && efd_full && NO > 0);
    if (n < 1 || n > 16) return DL_ERR_UNSUPPORTED;
    const int64_t items = NO * n;
    const int blocks = (int)(items < (int64_t)DL_NUM_SMS * 16 ? items : (int64_t)DL_NUM_SMS * 16);
    dwn_prepare_full_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(tables, efd_full, NO, (int)n, alpha, beta);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_fwd_bits_t(const uint32_t* in_bits_t, const int32_t* map, const uint64_t* masks,
                                uint32_t* out_bits_t, int64_t N, int64_t n, int64_t Bp,
                                dl_stream_t stream) {
    DL_REQUIRE(in_bits_t && map && masks && out_bits_t && N > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(in_bits_t, 16);
    DL_REQUIRE_ALIGNED(out_bits_t, 16);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int64_t Wp = Bp / 32;
    const int blocks = grid_for(N * (Wp / 4), 256);
    cudaStream_t s = dl_cast(stream);
    switch (n) {
        case 1: dwn_fwd_bits_kernel<1><<<blocks, 256, 0, s>>>(in_bits_t, map, masks, out_bits_t, N, Wp); break;
        case 2: dwn_fwd_bits_kernel<2><<<blocks, 256, 0, s>>>(in_bits_t, map, masks, out_bits_t, N, Wp); break;
        case 3: dwn_fwd_bits_kernel<3><<<blocks, 256, 0, s>>>(in_bits_t, map, masks, out_bits_t, N, Wp); break;
        case 4: dwn_fwd_bits_kernel<4><<<blocks, 256, 0, s>>>(in_bits_t, map, masks, out_bits_t, N, Wp); break;
        case 5: dwn_fwd_bits_kernel<5><<<blocks, 256, 0, s>>>(in_bits_t, map, masks, out_bits_t, N, Wp); break;
        default: dwn_fwd_bits_kernel<6><<<blocks, 256, 0, s>>>(in_bits_t, map, masks, out_bits_t, N, Wp); break;
    }
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_fwd_vals_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                                float* out_t, uint8_t* addr_t, int64_t N, int64_t n, int64_t Bp,
                                dl_stream_t stream) {
    DL_REQUIRE(in_bits_t && map && tables && out_t && N > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(out_t, 16);
    if (addr_t) DL_REQUIRE_ALIGNED(addr_t, 4);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int blocks = grid_for(N * (Bp / 128) * 32, 256);
    dwn_fwd_vals_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(in_bits_t, map, tables, out_t, addr_t, N,
                                                            (int)n, Bp);
    return dl_launch_status();
}

DL_EXPORT int64_t dl_dwn_groupsum_splits(int64_t N, int64_t k) {
    if (N <= 0 || k <= 0) return 1;
    const int64_t gsz = dl_ceil_div(N, k);
    int64_t s = gsz / 32;
    if (s < 1) s = 1;
    if (s > 16) s = 16;
    return s;
}

DL_EXPORT int dl_dwn_fwd_groupsum_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                                    float* partial, float* logits_t, int64_t N, int64_t n, int64_t k,
                                    float tau, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(in_bits_t && map && tables && partial && logits_t && N > 0 && k > 0 && tau > 0.f);
    DL_REQUIRE(Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(partial, 16);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int S = (int)dl_dwn_groupsum_splits(N, k);
    const int64_t gsz = dl_ceil_div(N, k);
    DL_REQUIRE(k * S <= 65535);
    dim3 grid((unsigned)dl_ceil_div(Bp, 512), (unsigned)(k * S));
    dwn_fwd_groupsum_kernel<<<grid, 128, 0, dl_cast(stream)>>>(in_bits_t, map, tables, partial, N, (int)n,
                                                              gsz, S, Bp);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    groupsum_reduce_kernel<<<grid_for(k * Bp, 256), 256, 0, dl_cast(stream)>>>(partial, logits_t, (int)k, S,
                                                                            1.0f / tau, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_bwd_tables_t(const uint32_t* in_bits_t, const int32_t* map, const float* g_t,
                                  int64_t gdiv, float gscale, float* gt, uint8_t* addr_t, int64_t N,
                                  int64_t n, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(in_bits_t && map && g_t && gt && N > 0 && gdiv > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(g_t, 16);
    if (addr_t) DL_REQUIRE_ALIGNED(addr_t, 4);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int64_t blocks64 = dl_ceil_div(N, HIST_WARPS);
    const int blocks = (int)(blocks64 < (int64_t)DL_NUM_SMS * 7 * 4 ? blocks64 : (int64_t)DL_NUM_SMS * 7 * 4);
    dwn_bwd_tables_kernel<<<blocks, HIST_WARPS * 32, 0, dl_cast(stream)>>>(in_bits_t, map, g_t, gdiv, gscale, gt,
                                                                          addr_t, N, (int)n, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_bwd_input_t(const uint8_t* addr_t, const float* g_t, int64_t gdiv, float gscale,
                                 const float* efd_t, const int32_t* inv_ptr, const int32_t* inv_ent,
                                 float* gx_t, int64_t F, int64_t n, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(addr_t && g_t && efd_t && inv_ptr && inv_ent && gx_t && F > 0 && gdiv > 0);
    DL_REQUIRE(Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(addr_t, 4);
    DL_REQUIRE_ALIGNED(g_t, 16);
    DL_REQUIRE_ALIGNED(gx_t, 16);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int blocks = grid_for(F * (Bp / 128) * 32, 256);
    dwn_bwd_input_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(addr_t, g_t, gdiv, gscale, efd_t, inv_ptr,
                                                             inv_ent, gx_t, F, (int)n, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_mapped_fwd(const float* xm, const float* tables, float* out, int64_t B, int64_t N,
                                int64_t n, int64_t O, int eval_mode, dl_stream_t stream) {
    DL_REQUIRE(xm && tables && out && B > 0 && N > 0 && O > 0);
    if (n < 1 || n > 16) return DL_ERR_UNSUPPORTED;
    dwn_mapped_fwd_kernel<<<grid_for(B * N, 256), 256, 0, dl_cast(stream)>>>(xm, tables, out, B, N, (int)n,
                                                                          (int)O, eval_mode != 0);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_mapped_bwd(const float* xm, const float* g, const float* efd_full, float* gxm,
                                float* gt, int64_t B, int64_t N, int64_t n, int64_t O,
                                dl_stream_t stream) {
    DL_REQUIRE(xm && g && B > 0 && N > 0 && O > 0 && (gxm || gt));
    if (n < 1 || n > 16) return DL_ERR_UNSUPPORTED;
    cudaStream_t s = dl_cast(stream);
    if (gxm != nullptr) {
        DL_REQUIRE(efd_full != nullptr);
        dwn_mapped_bwd_input_kernel<<<grid_for(B * N, 256), 256, 0, s>>>(xm, g, efd_full, gxm, B, N, (int)n,
                                                                      (int)O);
        if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    }
    if (gt != nullptr) {
        if (n <= DL_MAX_FAST_N) {
            const int64_t blocks = dl_ceil_div(N * O, 32);
            dwn_mapped_bwd_tables_kernel<<<(unsigned)blocks, HIST_WARPS * 32, 0, s>>>(xm, g, gt, B, N, (int)n,
                                                                                    (int)O);
        } else {
            if (cudaMemsetAsync(gt, 0, sizeof(float) * N * O * ((int64_t)1 << n), s) != cudaSuccess)
                return DL_ERR_LAUNCH;
            dwn_mapped_bwd_tables_atomic_kernel<<<grid_for(B * N, 256), 256, 0, s>>>(xm, g, gt, B, N, (int)n,
                                                                                  (int)O);
        }
    }
    return dl_launch_status();
}
