// DWN node kernels: LUT forward, extended-finite-difference (EFD) backward.
//
// Feature-major path ("_t"): activations are bit-packed [F][Bp/32]; a warp works on one node
// (or one input feature) and its lanes on consecutive samples, so every global access is a
// coalesced row segment.  Per sample the EFD backward is one address, one histogram update and
// n lookups in the per-step transform table `efd_t` instead of the reference's 2^n-term loop
// (difflut/nodes/dwn_node.py:195-227).
#include <cstdlib>
#include <mutex>

#include <cuda_bf16.h>

#include "common.cuh"

namespace {

// ------------------------------------------------------------------------------------------
// per-step table preparation
// ------------------------------------------------------------------------------------------

// One warp per node j (8 warps per CTA), looping over the slots i.  The 2^n table values sit two per lane (address
// = lane and lane+32) and go through the separable transform one address bit at a time: bit i
// becomes the difference (v1 - v0), every other bit b becomes v + beta * partner, where the
// partner differs in bit b only (a lane shuffle for bits 0..4, the lane's other register for bit
// 5).  The result does not depend on bit i of the address, so the entries with bit i = 0 are
// compacted into efd_t[j][i][0..2^(n-1)).  The same warp ballots the >= 0.5 masks.
template <int NIN>  // compile-time n (loops fully unrolled), or 0 to use the runtime value
__global__ void __launch_bounds__(256)
dwn_prepare_kernel(const float* __restrict__ tables, float* __restrict__ efd_t,
                   uint64_t* __restrict__ masks, int N, int n_rt, float alpha, float beta) {
    const int n = NIN > 0 ? NIN : n_rt;
    const int lane = threadIdx.x & 31;
    const int L = 1 << n;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int j = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; j < N; j += nwarps) {
        const float t_lo = lane < L ? __ldg(tables + (int64_t)j * L + lane) : 0.f;
        const float t_hi = lane + 32 < L ? __ldg(tables + (int64_t)j * L + lane + 32) : 0.f;
        if (masks != nullptr) {
            const uint32_t lo = __ballot_sync(0xffffffffu, lane < L && t_lo >= 0.5f);
            const uint32_t hi = __ballot_sync(0xffffffffu, lane + 32 < L && t_hi >= 0.5f);
            if (lane == 0) masks[j] = ((uint64_t)hi << 32) | lo;
        }
        if (efd_t == nullptr) continue;
#pragma unroll
        for (int i = 0; i < (NIN > 0 ? NIN : DL_MAX_FAST_N); ++i) {
            if (i >= n) break;
            float lo = alpha * t_lo, hi = alpha * t_hi;
#pragma unroll
            for (int b = 0; b < 5; ++b) {
                if (b >= n) break;
                const float plo = __shfl_xor_sync(0xffffffffu, lo, 1 << b);
                const float phi = __shfl_xor_sync(0xffffffffu, hi, 1 << b);
                if (b == i) {
                    const bool one = (lane >> b) & 1;
                    lo = one ? lo - plo : plo - lo;
                    hi = one ? hi - phi : phi - hi;
                } else {
                    lo = fmaf(beta, plo, lo);
                    hi = fmaf(beta, phi, hi);
                }
            }
            if (n == 6) {
                const float l0 = lo, h0 = hi;
                if (i == 5) {
                    lo = h0 - l0;
                    hi = h0 - l0;
                } else {
                    lo = fmaf(beta, h0, l0);
                    hi = fmaf(beta, l0, h0);
                }
            }
            // compact: keep addresses whose bit i is 0 and drop that bit
            float* dst = efd_t + ((int64_t)j * n + i) * 32;
            const int low = (1 << i) - 1;
            if (i == 5) {
                dst[lane] = lo;
            } else {
                if (lane < L && !((lane >> i) & 1)) {
                    const int a5 = ((lane >> (i + 1)) << i) | (lane & low);
                    dst[a5] = lo;
                    if (n == 6) dst[a5 + 16] = hi;
                }
                if (n < 6 && lane >= (L >> 1)) dst[lane] = 0.f;  // rows beyond 2^(n-1) are defined as zero
            }
        }
    }
}

// Transform with an arbitrary weight per Hamming distance (e.g. 1/(h+1) of the gradient-stabilised
// DWN variant, difflut/nodes/dwn_stable_node.py:170-202), which is not separable: thread (i, a') of a
// CTA evaluates the 2^n-term sum directly.  One CTA per node.
struct HammingWeights {
    float w[DL_MAX_FAST_N];
};

__global__ void __launch_bounds__(192)
dwn_prepare_weighted_kernel(const float* __restrict__ tables, float* __restrict__ efd_t,
                            uint64_t* __restrict__ masks, int N, int n, float scale, HammingWeights hw) {
    __shared__ float lut[64];
    const int L = 1 << n;
    for (int j = blockIdx.x; j < N; j += gridDim.x) {
        __syncthreads();
        if (threadIdx.x < 64) lut[threadIdx.x] = threadIdx.x < L ? __ldg(tables + (int64_t)j * L + threadIdx.x) : 0.f;
        __syncthreads();
        if (masks != nullptr && threadIdx.x < 32) {
            const int lane = threadIdx.x;
            const uint32_t lo = __ballot_sync(0xffffffffu, lane < L && lut[lane] >= 0.5f);
            const uint32_t hi = __ballot_sync(0xffffffffu, lane + 32 < L && lut[lane + 32] >= 0.5f);
            if (lane == 0) masks[j] = ((uint64_t)hi << 32) | lo;
        }
        if (efd_t == nullptr) continue;
        const int i = threadIdx.x >> 5, a5 = threadIdx.x & 31;
        if (i < n) {
            // slowly decaying weights leave a heavily cancelling +- sum: accumulate it in double (the
            // reference sums in Python floats, dwn_stable_node.py:178-200); this kernel is off the hot loop
            double acc = 0.0;
            if (a5 < (L >> 1)) {
                const int low = (1 << i) - 1;
                const int a = ((a5 & ~low) << 1) | (a5 & low);  // address with bit i = 0
                const int keep = (L - 1) & ~(1 << i);
                for (int k = 0; k < L; ++k) {
                    const double term = (double)lut[k] * (double)hw.w[__popc((a ^ k) & keep)];
                    acc += ((k >> i) & 1) ? term : -term;
                }
            }
            efd_t[((int64_t)j * n + i) * 32 + a5] = (float)((double)scale * acc);
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

// The multiplier and addend of leaf `p` of a node's multiplexer tree (see MuxTree): (t1 - t0, -t0).
__device__ __forceinline__ uint2 leaf_pair(uint64_t m, int p) {
    const uint32_t t0 = (uint32_t)(m >> (2 * p)) & 1u, t1 = (uint32_t)(m >> (2 * p + 1)) & 1u;
    return make_uint2(t1 - t0, 0u - t0);
}

// Depth-first evaluation of the 2^n -> 1 multiplexer tree on 4 words (128 samples) at once.
// A leaf turns two adjacent truth-table bits into all-zero / all-one masks and selects with
// input 0; every inner node is one select on input LVL.  BASE and LVL are compile-time, so
// every shift is an immediate and the tree is 2^n - 1 three-input logic ops per word.
// SMEM: the leaves come ready-made from shared memory, expanded once per node by the warp, and they are
// evaluated as integer multiply-adds instead of logic ops: with table bits (t0, t1) a leaf is 0, s, ~s or
// ~0, which is s * (t1 - t0) - t0 in 32-bit arithmetic (~s = -s - 1), so cm[p] = (t1 - t0, -t0) for table bits
// 2p and 2p+1.  The kernels are bound by the integer-logic pipe (measured 78-81 % busy with all 63 selects of
// a word on it); the 32 leaves of a word now go to the multiply-add pipe and 31 selects stay.
template <int LVL, int BASE, bool SMEM>
struct MuxTree {
    __device__ __forceinline__ static void eval(uint32_t lo, uint32_t hi, const uint2* cm, const uint4* x, uint4& out) {
        uint4 a, b;
        MuxTree<LVL - 1, BASE, SMEM>::eval(lo, hi, cm, x, a);
        MuxTree<LVL - 1, BASE + (1 << LVL), SMEM>::eval(lo, hi, cm, x, b);
        const uint4 s = x[LVL];
        out.x = (a.x & ~s.x) | (b.x & s.x);
        out.y = (a.y & ~s.y) | (b.y & s.y);
        out.z = (a.z & ~s.z) | (b.z & s.z);
        out.w = (a.w & ~s.w) | (b.w & s.w);
    }
};
template <int BASE, bool SMEM>
struct MuxTree<0, BASE, SMEM> {
    __device__ __forceinline__ static void eval(uint32_t lo, uint32_t hi, const uint2* cm, const uint4* x, uint4& out) {
        const uint4 s = x[0];
        if (SMEM) {
            const uint2 c = cm[BASE >> 1];
            out.x = s.x * c.x + c.y;
            out.y = s.y * c.x + c.y;
            out.z = s.z * c.x + c.y;
            out.w = s.w * c.x + c.y;
            return;
        }
        const uint32_t word = BASE < 32 ? lo : hi;
        const uint32_t c0 = 0u - ((word >> (BASE & 31)) & 1u);
        const uint32_t c1 = 0u - ((word >> ((BASE + 1) & 31)) & 1u);
        out.x = (c0 & ~s.x) | (c1 & s.x);
        out.y = (c0 & ~s.y) | (c1 & s.y);
        out.z = (c0 & ~s.z) | (c1 & s.z);
        out.w = (c0 & ~s.w) | (c1 & s.w);
    }
};

// Thread (x = group of 4 words, y = node): consecutive x read contiguous 16-byte pieces of each
// input row.  Node tiles are the fast grid dimension and word-group tiles the slow one, so the CTAs
// resident at any time work on one slab of the batch (its input rows stay in L2 while all nodes
// gather from them); both are walked with grid-stride loops (no index division).
// SMEM needs blockDim.x to be a multiple of 32, so that all lanes of a warp work on the same node.
template <int NIN, bool SMEM>
__global__ void __launch_bounds__(256, 4)
dwn_fwd_bits_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                    const uint64_t* __restrict__ masks, uint32_t* __restrict__ out_bits, int N, int Q) {
    __shared__ uint2 cm_all[SMEM ? 8 : 1][32];
    const int tid = threadIdx.y * blockDim.x + threadIdx.x;
    const int lane = tid & 31;
    uint2* cm = cm_all[SMEM ? (tid >> 5) : 0];
    const int64_t Wp = (int64_t)Q << 2;
    // SMEM: the word-group loop runs to a warp-uniform bound so that whole warps reach the __syncwarp
    const int qend = SMEM ? ((Q + 31) & ~31) : Q;
    for (int q = blockIdx.y * blockDim.x + threadIdx.x; q < qend; q += gridDim.y * blockDim.x) {
        for (int j = blockIdx.x * blockDim.y + threadIdx.y; j < N; j += gridDim.x * blockDim.y) {
            const uint64_t m = __ldg(&masks[j]);
            if (SMEM) {
                __syncwarp();
                cm[lane] = leaf_pair(m, lane);
                __syncwarp();
                if (q >= Q) continue;
            }
            uint4 x[NIN];
#pragma unroll
            for (int i = 0; i < NIN; ++i)
                x[i] = __ldg(reinterpret_cast<const uint4*>(in_bits + (int64_t)__ldg(&map[j * NIN + i]) * Wp) + q);
            uint4 o;
            MuxTree<NIN - 1, 0, SMEM>::eval((uint32_t)m, (uint32_t)(m >> 32), cm, x, o);
            reinterpret_cast<uint4*>(out_bits + (int64_t)j * Wp)[q] = o;
        }
    }
}

// The same layer as a persistent kernel for batches of whole 4096-sample tiles.  A warp walks items
// (tile of 32 word groups, node), tile-major so that the warps of the grid share one slab of input rows.
// Two stages of loads run ahead of the multiplexer tree: the index row and leaf mask of the item after next
// (one value per lane, handed out by shuffles) and the six 16-byte pieces of the next item, so the tree of
// one item (128 multiply-adds and 124 selects per thread) never waits for a dependent pair of L2 round trips.
// The two register sets swap roles every item (the loop body is written out twice), so nothing is copied.
constexpr int FWD_STREAM_WARPS = 8;

template <int NIN, int CTAS>
__global__ void __launch_bounds__(FWD_STREAM_WARPS * 32, CTAS)
dwn_fwd_bits_stream_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                           const uint64_t* __restrict__ masks, uint32_t* __restrict__ out_bits, int N, int Q) {
    __shared__ uint2 cm_all[FWD_STREAM_WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint2* cm = cm_all[warp];
    const int64_t Wp = (int64_t)Q << 2;
    const uint32_t tiles = (uint32_t)Q >> 5, nodes = (uint32_t)N;
    const uint32_t stride = gridDim.x * FWD_STREAM_WARPS;
    const uint32_t* masks32 = reinterpret_cast<const uint32_t*>(masks);

    // the frontier of the item sequence of this warp: (tile tf, node jf)
    uint32_t tf, jf;
    {
        const uint32_t first = blockIdx.x * FWD_STREAM_WARPS + warp;
        tf = first / nodes;
        jf = first - tf * nodes;
    }
    // index data of the frontier item, one value per lane (lanes 0..NIN-1 the input rows, then the two halves
    // of the leaf mask); afterwards the frontier moves on by one stride
    auto take = [&](uint32_t& j, uint32_t& q, uint32_t& meta) -> bool {
        const bool ok = tf < tiles;
        j = jf;
        q = tf * 32 + lane;
        meta = 0;
        if (ok) {
            if (lane < NIN) meta = (uint32_t)__ldg(&map[jf * NIN + lane]);
            else if (lane < NIN + 2) meta = __ldg(&masks32[2 * jf + (lane - NIN)]);
        }
        jf += stride;
        while (jf >= nodes) {
            jf -= nodes;
            ++tf;
        }
        return ok;
    };
    auto load_x = [&](uint4 (&x)[NIN], uint32_t meta, uint32_t q) {
#pragma unroll
        for (int i = 0; i < NIN; ++i) {
            const uint32_t row = __shfl_sync(0xffffffffu, meta, i);
            x[i] = __ldg(reinterpret_cast<const uint4*>(in_bits + (int64_t)row * Wp) + q);
        }
    };
    auto compute = [&](const uint4 (&x)[NIN], uint32_t meta, uint32_t j, uint32_t q) {
        const uint32_t lo = __shfl_sync(0xffffffffu, meta, NIN), hi = __shfl_sync(0xffffffffu, meta, NIN + 1);
        __syncwarp();  // the previous item's leaves are no longer read
        cm[lane] = leaf_pair(((uint64_t)hi << 32) | lo, lane);
        __syncwarp();
        uint4 o;
        MuxTree<NIN - 1, 0, true>::eval(lo, hi, cm, x, o);
        reinterpret_cast<uint4*>(out_bits + (int64_t)j * Wp)[q] = o;
    };

    uint4 xa[NIN], xb[NIN];
    uint32_t ja, qa, ma, jb, qb, mb, jc, qc, mc;
    if (!take(ja, qa, ma)) return;
    bool okb = take(jb, qb, mb);
    load_x(xa, ma, qa);
    while (true) {
        bool okc = take(jc, qc, mc);           // two items ahead: index data
        if (okb) load_x(xb, mb, qb);           // one item ahead: input words
        compute(xa, ma, ja, qa);
        if (!okb) break;
        okb = take(ja, qa, ma);
        if (okc) load_x(xa, mc, qc);
        compute(xb, mb, jb, qb);
        if (!okc) break;
        // roles for the next round: a = the item whose words were just requested, b = the one whose index data was
        jb = ja; qb = qa; mb = ma;
        ja = jc; qa = qc; ma = mc;
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

// Training forward, one warp per (1024-sample slab, node); lane = 4 consecutive samples of each
// 128-sample chunk.  Slabs are the outer order, so the warps of the grid share one slab of input rows
// at a time and layers with few nodes still fill the machine.
__global__ void __launch_bounds__(256)
dwn_fwd_vals_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                    const float* __restrict__ tables, float* __restrict__ out_t,
                    uint8_t* __restrict__ addr_t, int64_t N, int n, int64_t Bp) {
    const int lane = threadIdx.x & 31;
    const int64_t C = Bp >> 7, Wp = Bp >> 5;
    const int64_t G = (C + 7) >> 3;
    const int L = 1 << n;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < G * N; item += nwarps) {
        const int64_t cg = item / N, j = item - cg * N;
        int32_t rows[DL_MAX_FAST_N];
#pragma unroll
        for (int i = 0; i < DL_MAX_FAST_N; ++i) rows[i] = i < n ? __ldg(&map[j * n + i]) : 0;
        const float* tj = tables + j * L;
        const int64_t c1 = (cg + 1) * 8 < C ? (cg + 1) * 8 : C;
        for (int64_t c = cg * 8; c < c1; ++c) {
            const int64_t b = (c << 7) + lane * 4;
            const uint32_t a = addr4(in_bits, rows, n, Wp, b);
            float4 o;
            o.x = __ldg(tj + (a & 0xFF));
            o.y = __ldg(tj + ((a >> 8) & 0xFF));
            o.z = __ldg(tj + ((a >> 16) & 0xFF));
            o.w = __ldg(tj + (a >> 24));
            *reinterpret_cast<float4*>(out_t + j * Bp + b) = o;
            if (addr_t != nullptr) *reinterpret_cast<uint32_t*>(addr_t + j * Bp + b) = a;
        }
    }
}

// Last layer fused with GroupSum.  One CTA per (1024-sample group, class*S + slice); its 4 warps
// share the slice's nodes (warp w takes nodes w, w+4, ...) and add their sums through shared memory
// in a fixed order.  For each node lane w loads word w of the node's 6 input rows (coalesced), the 8
// chunks of the group get their words by shuffle, and 32 running sums (8 chunks x 4 samples) stay
// in registers; the next node's words are loaded before the current node is consumed.
// SWZ: chunk-interleaved input bits (see dl_bits_swizzle_t): the lane's own word holds its samples.
// NFIX: the node width as a compile-time constant (0 = read it from `n_arg`), which removes the per-input
// predicates from the address formation.
template <bool SWZ, int NFIX>
__global__ void __launch_bounds__(128)
dwn_fwd_groupsum_kernel(const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                        const float* __restrict__ tables, float* __restrict__ partial, int64_t N,
                        int n_arg, int64_t gsz, int S, int64_t Bp, int64_t Wp) {
    __shared__ float4 red[3][8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = NFIX > 0 ? NFIX : n_arg;
    const int L = 1 << n;
    const int64_t grp = blockIdx.x;  // 1024-sample group
    const int64_t cls = blockIdx.y / (unsigned)S, s = blockIdx.y % (unsigned)S;
    const int64_t per = (gsz + S - 1) / S;
    const int64_t j0 = cls * gsz + s * per;
    int64_t j1 = j0 + per;
    if (j1 > (cls + 1) * gsz) j1 = (cls + 1) * gsz;
    if (j1 > N) j1 = N;
    const int64_t w = grp * 32 + lane;
    const bool wvalid = w < Wp;
    const int src_lane = lane >> 3, sh = (lane & 7) * 4;
    float4 acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t nxt[DL_MAX_FAST_N];
    const int64_t jfirst = j0 + warp;
#pragma unroll
    for (int i = 0; i < DL_MAX_FAST_N; ++i)
        nxt[i] = (i < n && jfirst < j1 && wvalid) ? __ldg(in_bits + (int64_t)__ldg(&map[jfirst * n + i]) * Wp + w) : 0u;
    for (int64_t j = jfirst; j < j1; j += 4) {
        uint32_t words[DL_MAX_FAST_N];
#pragma unroll
        for (int i = 0; i < DL_MAX_FAST_N; ++i) words[i] = nxt[i];
        if (j + 4 < j1) {
#pragma unroll
            for (int i = 0; i < DL_MAX_FAST_N; ++i)
                nxt[i] = (i < n && wvalid) ? __ldg(in_bits + (int64_t)__ldg(&map[(j + 4) * n + i]) * Wp + w) : 0u;
        }
        const char* tj = reinterpret_cast<const char*>(tables + j * L);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            // four table offsets in bytes, one per byte of `a` (addresses < 64, so address * 4 stays inside its byte)
            uint32_t a = 0;
#pragma unroll
            for (int i = 0; i < DL_MAX_FAST_N; ++i) {
                if (i < n) {
                    if (SWZ) {
                        const uint32_t t = c >= i + 2 ? words[i] >> (c - i - 2) : words[i] << (i + 2 - c);
                        a |= t & (0x04040404u << i);
                    } else {
                        const uint32_t t = __shfl_sync(0xffffffffu, words[i], c * 4 + src_lane) >> sh;
                        a |= dl_spread_nibble(t & 0xFu) << (i + 2);
                    }
                }
            }
            // one byte extract and one 64-bit add per look-up
            acc[c].x += __ldg(reinterpret_cast<const float*>(tj + __byte_perm(a, 0, 0x4440)));
            acc[c].y += __ldg(reinterpret_cast<const float*>(tj + __byte_perm(a, 0, 0x4441)));
            acc[c].z += __ldg(reinterpret_cast<const float*>(tj + __byte_perm(a, 0, 0x4442)));
            acc[c].w += __ldg(reinterpret_cast<const float*>(tj + __byte_perm(a, 0, 0x4443)));
        }
    }
    if (warp > 0) {
#pragma unroll
        for (int c = 0; c < 8; ++c) red[warp - 1][c][lane] = acc[c];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
#pragma unroll
            for (int o = 0; o < 3; ++o) {
                const float4 v = red[o][c][lane];
                acc[c].x += v.x; acc[c].y += v.y; acc[c].z += v.z; acc[c].w += v.w;
            }
            const int64_t b = grp * 1024 + c * 128 + lane * 4;
            if (b < Bp) *reinterpret_cast<float4*>(partial + (int64_t)blockIdx.y * Bp + b) = acc[c];
        }
    }
}

__global__ void groupsum_reduce_kernel(const float* __restrict__ partial, float* __restrict__ logits_t,
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

// The same reduction followed at once by the mean cross-entropy of the logits (the arithmetic of ce_t_kernel in
// head.cu, same order: identical bits), one launch instead of two on the path from the last layer to the
// backward kernels.  A CTA takes 32 samples; thread (class lane cl, sample lane) reduces the partial sums of
// the classes cl, cl + 8, ... and leaves the logits in shared memory; the first warp then does the softmax
// of its 32 samples.  k <= CE_MAX_CLASSES.
constexpr int CE_MAX_CLASSES = 128;

__global__ void __launch_bounds__(256)
groupsum_reduce_ce_kernel(const float* __restrict__ partial, float* __restrict__ logits_t,
                          const int32_t* __restrict__ labels, float* __restrict__ dlogits_t,
                          float* __restrict__ loss_rows, int k, int S, float inv_tau, int64_t B, float inv_bg,
                          int64_t Bp) {
    extern __shared__ float lg[];  // [k][32]
    const int lane = threadIdx.x & 31, cl = threadIdx.x >> 5;
    for (int64_t b0 = (int64_t)blockIdx.x * 32; b0 < Bp; b0 += (int64_t)gridDim.x * 32) {
        const int64_t b = b0 + lane;
        __syncthreads();  // the previous 32 samples' logits are no longer read
        for (int c = cl; c < k; c += 8) {
            // eight loads in flight at a time; the additions keep their order, so the sum is unchanged
            const float* src = partial + (int64_t)c * S * Bp + b;
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
            const float logit = acc * inv_tau;
            logits_t[(int64_t)c * Bp + b] = logit;
            lg[c * 32 + lane] = logit;
        }
        __syncthreads();
        if (cl != 0) continue;
        if (b >= B) {
            for (int c = 0; c < k; ++c) dlogits_t[(int64_t)c * Bp + b] = 0.f;
            loss_rows[b] = 0.f;
            continue;
        }
        float mx = -INFINITY;
        for (int c = 0; c < k; ++c) mx = fmaxf(mx, lg[c * 32 + lane]);
        float sum = 0.f;
        for (int c = 0; c < k; ++c) sum += expf(lg[c * 32 + lane] - mx);
        const float lse = mx + logf(sum);
        const int y = labels[b];
        if (y < 0 || y >= k) {  // no such class: no gradient, NaN loss (see dl_ce_t)
            for (int c = 0; c < k; ++c) dlogits_t[(int64_t)c * Bp + b] = 0.f;
            loss_rows[b] = __int_as_float(0x7fc00000);
            continue;
        }
        const float inv = 1.0f / sum;
        for (int c = 0; c < k; ++c) {
            const float p = expf(lg[c * 32 + lane] - mx) * inv;
            dlogits_t[(int64_t)c * Bp + b] = (p - (c == y ? 1.f : 0.f)) * inv_bg;
        }
        loss_rows[b] = lse - lg[y * 32 + lane];
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
        const float* grow = g_t + (gdiv == 1 ? j : (int64_t)((uint32_t)j / (uint32_t)gdiv)) * Bp;
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
                     float* __restrict__ gx_t, int64_t F, int n, int64_t Bp, int cps) {
    constexpr int CH = 4;  // chunks per work item: a reader's index data is loaded once per 512 samples
    const int lane = threadIdx.x & 31;
    const int64_t C = Bp >> 7;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    // The batch is walked in passes of `cps` chunks (a multiple of 8: whole 1024-sample slabs); inside a
    // pass one warp owns one (feature, 4 chunks) item and the items of a feature go to neighbouring warps.
    // With many features a pass is one slab, so the slab of g_t / addr_t the warps share stays in L2;
    // with few features (a convolution's patch taps) the host widens the pass until every warp has work.
    // Per reader the item's four address words and gradient pieces are requested together.
    const uint32_t ugdiv = (uint32_t)gdiv;
    const int ipp = cps / CH;  // items of a feature per pass
    const int64_t items = F * ipp;
    for (int64_t c0 = 0; c0 < C; c0 += cps)
    for (int64_t it = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; it < items; it += nwarps) {
        const int64_t f = it / ipp;
        const int64_t cb = c0 + (it - f * ipp) * CH;
        if (cb >= C) continue;  // uniform over the warp
        const int64_t b = (cb << 7) + lane * 4;
        const int e0 = __ldg(&inv_ptr[f]), e1 = __ldg(&inv_ptr[f + 1]);
        float4 acc[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int e = e0; e < e1; ++e) {
            const int ent = __ldg(&inv_ent[e]);
            const int j = ent >> 3, i = ent & 7;
            const float tv = __ldg(efd_t + ((int64_t)j * n + i) * 32 + lane);
            const int64_t grow = ugdiv == 1 ? j : (int64_t)((uint32_t)j / ugdiv);
            uint32_t a[CH];
            float4 g[CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const bool live = cb + c < C;
                a[c] = live ? __ldg(reinterpret_cast<const uint32_t*>(addr_t + (int64_t)j * Bp + b + c * 128)) : 0u;
                g[c] = live ? __ldg(reinterpret_cast<const float4*>(g_t + grow * Bp + b + c * 128))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            const uint32_t low = (1u << i) - 1u;
            // drop bit i of every byte: keep the bits below i, shift the bits above i down by one
            const uint32_t lowm = low * 0x01010101u;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const uint32_t a5 = (a[c] & lowm) | ((a[c] >> 1) & ~lowm & 0x7F7F7F7Fu);
                acc[c].x += g[c].x * __shfl_sync(0xffffffffu, tv, a5 & 31);
                acc[c].y += g[c].y * __shfl_sync(0xffffffffu, tv, (a5 >> 8) & 31);
                acc[c].z += g[c].z * __shfl_sync(0xffffffffu, tv, (a5 >> 16) & 31);
                acc[c].w += g[c].w * __shfl_sync(0xffffffffu, tv, (a5 >> 24) & 31);
            }
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            if (cb + c < C) {
                acc[c].x *= gscale; acc[c].y *= gscale; acc[c].z *= gscale; acc[c].w *= gscale;
                *reinterpret_cast<float4*>(gx_t + f * Bp + b + c * 128) = acc[c];
            }
        }
    }
}

// The same input gradient for a connection map in which no input feature has more than one reader (the
// identity map a LearnableLayer's soft selection feeds: node j reads features j*n .. j*n+n-1).  Nothing has to
// be summed, so the work is turned around: one warp per (node, 1024-sample slab) loads the node's gradient and
// addresses once and writes its n input-gradient rows, instead of one warp per (feature, chunk) chasing the
// inverse map through four dependent loads.  BF16: the rows leave as bf16 (round to nearest), which is what the
// weight-gradient contraction of the soft selection reads.
template <bool BF16>
__global__ void __launch_bounds__(256)
dwn_bwd_input_disjoint_kernel(const uint8_t* __restrict__ addr_t, const float* __restrict__ g_t, uint32_t ugdiv,
                              float gscale, const float* __restrict__ efd_t, const int32_t* __restrict__ map,
                              void* __restrict__ out, int64_t NO, int n, int64_t Bp) {
    const int lane = threadIdx.x & 31;
    const int64_t C = Bp >> 7, G = (C + 7) >> 3;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < G * NO; item += nwarps) {
        const int64_t cg = item / NO, j = item - cg * NO;
        float tv[DL_MAX_FAST_N];
        int64_t row[DL_MAX_FAST_N];
#pragma unroll
        for (int i = 0; i < DL_MAX_FAST_N; ++i) {
            tv[i] = i < n ? gscale * __ldg(efd_t + (j * n + i) * 32 + lane) : 0.f;
            row[i] = i < n ? (int64_t)__ldg(map + j * n + i) : 0;
        }
        const int64_t grow = ugdiv == 1 ? j : (int64_t)((uint32_t)j / ugdiv);
        const int64_t c1 = (cg + 1) * 8 < C ? (cg + 1) * 8 : C;
        for (int64_t c = cg * 8; c < c1; ++c) {
            const int64_t b = (c << 7) + lane * 4;
            const uint32_t a = __ldg(reinterpret_cast<const uint32_t*>(addr_t + j * Bp + b));
            const float4 g = __ldg(reinterpret_cast<const float4*>(g_t + grow * Bp + b));
#pragma unroll
            for (int i = 0; i < DL_MAX_FAST_N; ++i) {
                if (i < n) {
                    const uint32_t lowm = ((1u << i) - 1u) * 0x01010101u;
                    const uint32_t a5 = (a & lowm) | ((a >> 1) & ~lowm & 0x7F7F7F7Fu);
                    float4 r;
                    r.x = g.x * __shfl_sync(0xffffffffu, tv[i], a5);
                    r.y = g.y * __shfl_sync(0xffffffffu, tv[i], a5 >> 8);
                    r.z = g.z * __shfl_sync(0xffffffffu, tv[i], a5 >> 16);
                    r.w = g.w * __shfl_sync(0xffffffffu, tv[i], a5 >> 24);
                    if (BF16) {
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
                        uint2 pk;
                        pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                        pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + row[i] * Bp + b) = pk;
                    } else {
                        *reinterpret_cast<float4*>(static_cast<float*>(out) + row[i] * Bp + b) = r;
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// fused backward of one layer: output gradient (pulled from the layer above) + table gradient
// ------------------------------------------------------------------------------------------

constexpr int FUSED_CG = 8;  // 128-sample chunks per work item (1024 samples)

// One warp per (1024-sample group cg, node f of THIS layer).  Step 1 forms the gradient w.r.t. the
// node's output for the 8 chunks of the group: either read directly (DIRECT: g_up rows, e.g. the
// GroupSum gradient) or pulled from the layer above through the inverse map, exactly as
// dwn_bwd_input_kernel does.  Step 2 forms the node's own addresses from its input bits and adds
// the gradients into a lane-private histogram, which is written as one partial table gradient per
// (group, node); the caller sums the groups in order (dl_sum_groups).  The output gradient and the
// addresses are stored only when the layer below needs them, so for the first layer its
// [N][Bp] fp32 gradient never reaches HBM.
constexpr int FUSED_MAX_REG_CONTRIB = 3;  // inverse-map entries of a node kept in registers

// T-table lookups of 4 samples: the lane index of each shuffle is the sample's address without
// bit i (a shuffle takes its source lane modulo 32, so the bytes above need no masking).
__device__ __forceinline__ void efd_accumulate(float4& acc, const float4 g, const uint32_t a, const uint32_t lowm,
                                               const float tv) {
    const uint32_t a5 = (a & lowm) | ((a >> 1) & ~lowm & 0x7F7F7F7Fu);
    acc.x = fmaf(g.x, __shfl_sync(0xffffffffu, tv, a5), acc.x);
    acc.y = fmaf(g.y, __shfl_sync(0xffffffffu, tv, a5 >> 8), acc.y);
    acc.z = fmaf(g.z, __shfl_sync(0xffffffffu, tv, a5 >> 16), acc.z);
    acc.w = fmaf(g.w, __shfl_sync(0xffffffffu, tv, a5 >> 24), acc.w);
}

// Data one chunk needs from the layer above: CNT (address word, gradient float4) pairs, or one
// gradient float4 in DIRECT mode.  Loads are issued unconditionally (no branch between them) so that
// they overlap; the next chunk's loads are issued before the current chunk is consumed.
// CNT = 0..3: exactly that many readers, all in registers; CNT = 4: three in registers plus `extra`
// more walked through the inverse map; CNT = 5: none in registers, all `extra` readers walked.
template <int CNT>
struct ChunkData {
    static constexpr int REG = CNT == 5 ? 0 : (CNT > FUSED_MAX_REG_CONTRIB ? FUSED_MAX_REG_CONTRIB : CNT);
    uint32_t a[REG > 0 ? REG : 1];
    float4 g[REG > 0 ? REG : 1];
};

template <bool DIRECT, int CNT>
__device__ __forceinline__ void load_chunk(ChunkData<CNT>& d, int c, const float* __restrict__ gdir,
                                           const uint8_t* const (&ap)[FUSED_MAX_REG_CONTRIB],
                                           const float* const (&gp)[FUSED_MAX_REG_CONTRIB]) {
    if (DIRECT) {
        d.g[0] = __ldg(reinterpret_cast<const float4*>(gdir + c * 128));
    } else {
#pragma unroll
        for (int k = 0; k < ChunkData<CNT>::REG; ++k) {
            d.a[k] = __ldg(reinterpret_cast<const uint32_t*>(ap[k] + c * 128));
            d.g[k] = __ldg(reinterpret_cast<const float4*>(gp[k] + c * 128));
        }
    }
}

// Everything chunk c does once its data is in registers: output gradient, own addresses, stores,
// histogram update.  NIN is the compile-time node input count (0 = use the runtime value n).
// SWZ: the input bits are in the chunk-interleaved layout (bit c + 8r of word w of a 1024-sample
// block = sample 128c + 4w + r), so the lane's own word already holds its four samples of chunk c one
// per byte and an address bit costs a shift and a masked or.  OUTS: bit 0 = store the output gradient,
// bit 1 = store the addresses (-1: decide at run time from the pointers).
template <bool DIRECT, int CNT, int NIN, bool SWZ, int OUTS>
__device__ __forceinline__ void consume_chunk(
    const ChunkData<CNT>& d, int c, int n, int extra, int src_lane, int sh, float gscale,
    const uint32_t (&words)[DL_MAX_FAST_N], const float (&tv)[FUSED_MAX_REG_CONTRIB],
    const uint32_t (&lowm)[FUSED_MAX_REG_CONTRIB], const int32_t* __restrict__ inv_ent, int e_tail,
    const uint8_t* __restrict__ addr_up, const float* __restrict__ g_up, const float* __restrict__ efd_up,
    int n_up, uint32_t ugdiv, int64_t Bp, int64_t b0, float* __restrict__ go, uint8_t* __restrict__ ao,
    float* __restrict__ mine) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (DIRECT) {
        acc = d.g[0];
        acc.x *= gscale; acc.y *= gscale; acc.z *= gscale; acc.w *= gscale;
    } else {
#pragma unroll
        for (int k = 0; k < ChunkData<CNT>::REG; ++k) efd_accumulate(acc, d.g[k], d.a[k], lowm[k], tv[k]);
        if (CNT > FUSED_MAX_REG_CONTRIB)
        for (int k = 0; k < extra; ++k) {  // rare: more readers than registers
            const int ent = __ldg(&inv_ent[e_tail + k]);
            const int j = ent >> 3, i = ent & 7;
            const float t = gscale * __ldg(efd_up + ((int64_t)j * n_up + i) * 32 + (threadIdx.x & 31));
            const int64_t b = b0 + c * 128;
            const uint32_t a = __ldg(reinterpret_cast<const uint32_t*>(addr_up + (int64_t)j * Bp + b));
            const int64_t gr = ugdiv == 1 ? (int64_t)j : (int64_t)((uint32_t)j / ugdiv);
            const float4 g = __ldg(reinterpret_cast<const float4*>(g_up + gr * Bp + b));
            efd_accumulate(acc, g, a, ((1u << i) - 1u) * 0x01010101u, t);
        }
    }
    // own addresses: fetch the word of this lane's samples from the lane that loaded it
    uint32_t a = 0;
#pragma unroll
    for (int i = 0; i < DL_MAX_FAST_N; ++i) {
        if (NIN > 0 ? i < NIN : i < n) {
            if (SWZ) {
                const uint32_t t = c >= i ? words[i] >> (c - i) : words[i] << (i - c);
                a |= t & (0x01010101u << i);
            } else {
                const uint32_t t = __shfl_sync(0xffffffffu, words[i], c * 4 + src_lane) >> sh;
                a |= dl_spread_nibble(t & 0xFu) << i;
            }
        }
    }
    if (OUTS < 0 ? go != nullptr : (OUTS & 1) != 0) *reinterpret_cast<float4*>(go + c * 128) = acc;
    if (OUTS < 0 ? ao != nullptr : (OUTS & 2) != 0) *reinterpret_cast<uint32_t*>(ao + c * 128) = a;
    // bin e of this lane lives at float offset e*32: byte offset e << 7
    char* base = reinterpret_cast<char*>(mine);
    *reinterpret_cast<float*>(base + ((a << 7) & 0x1F80u)) += acc.x;
    *reinterpret_cast<float*>(base + ((a >> 1) & 0x1F80u)) += acc.y;
    *reinterpret_cast<float*>(base + ((a >> 9) & 0x1F80u)) += acc.z;
    *reinterpret_cast<float*>(base + ((a >> 17) & 0x1F80u)) += acc.w;
}

#define DL_CONSUME_ARGS n, extra, src_lane, sh, gscale, words, tv, lowm, inv_ent, e_tail, addr_up, g_up, efd_up, \
                        n_up, ugdiv, Bp, b0, go, ao, mine

// The chunks of one (group, node) item for a node with exactly CNT readers held in registers.
// FULL: all 8 chunks exist; they are processed as 4 unrolled pairs with two register buffers
// (ping-pong), so the loads of chunk c+1 fly while chunk c is consumed and nothing is copied.
template <bool DIRECT, int CNT, int NIN, bool FULL, bool SWZ, int OUTS>
__device__ __forceinline__ void fused_chunks(
    int valid_chunks, int n, int extra, int src_lane, int sh, float gscale, const uint32_t (&words)[DL_MAX_FAST_N],
    const float* __restrict__ gdir, const uint8_t* const (&ap)[FUSED_MAX_REG_CONTRIB],
    const float* const (&gp)[FUSED_MAX_REG_CONTRIB], const float (&tv)[FUSED_MAX_REG_CONTRIB],
    const uint32_t (&lowm)[FUSED_MAX_REG_CONTRIB], const int32_t* __restrict__ inv_ent, int e_tail,
    const uint8_t* __restrict__ addr_up, const float* __restrict__ g_up, const float* __restrict__ efd_up,
    int n_up, uint32_t ugdiv, int64_t Bp, int64_t b0, float* __restrict__ go, uint8_t* __restrict__ ao,
    float* __restrict__ mine) {
    if (FULL) {
        ChunkData<CNT> even, odd;
        load_chunk<DIRECT, CNT>(even, 0, gdir, ap, gp);
#pragma unroll
        for (int c = 0; c < FUSED_CG; c += 2) {
            load_chunk<DIRECT, CNT>(odd, c + 1, gdir, ap, gp);
            consume_chunk<DIRECT, CNT, NIN, SWZ, OUTS>(even, c, DL_CONSUME_ARGS);
            if (c + 2 < FUSED_CG) load_chunk<DIRECT, CNT>(even, c + 2, gdir, ap, gp);
            consume_chunk<DIRECT, CNT, NIN, SWZ, OUTS>(odd, c + 1, DL_CONSUME_ARGS);
        }
    } else {
        for (int c = 0; c < valid_chunks; ++c) {
            ChunkData<CNT> d;
            load_chunk<DIRECT, CNT>(d, c, gdir, ap, gp);
            consume_chunk<DIRECT, CNT, NIN, SWZ, OUTS>(d, c, DL_CONSUME_ARGS);
        }
    }
}
#undef DL_CONSUME_ARGS

template <bool DIRECT, int NIN, bool SWZ, int OUTS>
__global__ void __launch_bounds__(HIST_WARPS * 32, 5)
dwn_bwd_fused_kernel(const uint8_t* __restrict__ addr_up, const float* __restrict__ g_up, int64_t gdiv_up,
                     float gscale_up, const float* __restrict__ efd_up, int n_up,
                     const int32_t* __restrict__ inv_ptr, const int32_t* __restrict__ inv_ent,
                     const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                     float* __restrict__ g_out, uint8_t* __restrict__ addr_out,
                     float* __restrict__ gt_partial, int64_t group_stride, int64_t N, int n_rt, int64_t Bp,
                     int64_t Wp) {
    __shared__ __align__(16) float hist_all[HIST_WARPS][64 * 32];
    const int n = NIN > 0 ? NIN : n_rt;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* hist = hist_all[warp];      // hist[e * 32 + lane]: bin e, private to the lane
    float* mine = hist + lane;
    const int64_t C = Bp >> 7;  // Wp: words per input row (Bp/32, or 32 per 1024-sample block when SWZ)
    const int64_t G = (C + FUSED_CG - 1) / FUSED_CG;
    const int L = 1 << n;
    const int64_t nwarps = (int64_t)gridDim.x * HIST_WARPS;
    const uint32_t ugdiv = (uint32_t)gdiv_up;
    const int src_lane = lane >> 3;          // which of a chunk's 4 words holds this lane's samples
    const int sh = (lane & 7) * 4;           // bit offset of its 4 samples inside that word
    // gridDim.y > 1 only with one slab per group (group_stride > 0): the groups are then independent and
    // layers with few nodes spread them over the grid's second dimension
    for (int64_t cg = blockIdx.y; cg < G; cg += gridDim.y) {
        const int64_t left = C - cg * FUSED_CG;
        const int valid_chunks = left < FUSED_CG ? (int)left : FUSED_CG;
        for (int64_t f = (int64_t)blockIdx.x * HIST_WARPS + warp; f < N; f += nwarps) {
            const int64_t b0 = cg * (FUSED_CG * 128) + lane * 4;
            // this node's input words for the whole group: lane w holds word w of each input row
            uint32_t words[DL_MAX_FAST_N];
#pragma unroll
            for (int i = 0; i < DL_MAX_FAST_N; ++i) {
                words[i] = 0u;
                if (i < n) {
                    const int64_t w = cg * (FUSED_CG * 4) + lane;
                    if (w < Wp) words[i] = __ldg(in_bits + (int64_t)__ldg(&map[f * n + i]) * Wp + w);
                }
            }
            // inverse-map entries of this node: the first few stay in registers for all chunks; the
            // output-gradient scale is folded into their EFD values
            int e0 = 0, cnt = 0;
            float tv_r[FUSED_MAX_REG_CONTRIB];
            uint32_t lowm_r[FUSED_MAX_REG_CONTRIB];
            const uint8_t* ap[FUSED_MAX_REG_CONTRIB];
            const float* gp[FUSED_MAX_REG_CONTRIB];
            const float* gdir = nullptr;
            if (DIRECT) {
                gdir = g_up + (ugdiv == 1 ? f : (int64_t)((uint32_t)f / ugdiv)) * Bp + b0;
            } else {
                e0 = __ldg(&inv_ptr[f]);
                cnt = __ldg(&inv_ptr[f + 1]) - e0;
#pragma unroll
                for (int k = 0; k < FUSED_MAX_REG_CONTRIB; ++k) {
                    tv_r[k] = 0.f; lowm_r[k] = 0u; ap[k] = addr_up; gp[k] = g_up;
                    if (k < cnt) {
                        const int ent = __ldg(&inv_ent[e0 + k]);
                        const int j = ent >> 3, i = ent & 7;
                        tv_r[k] = gscale_up * __ldg(efd_up + ((int64_t)j * n_up + i) * 32 + lane);
                        lowm_r[k] = ((1u << i) - 1u) * 0x01010101u;
                        ap[k] = addr_up + (int64_t)j * Bp + b0;
                        gp[k] = g_up + (ugdiv == 1 ? (int64_t)j : (int64_t)((uint32_t)j / ugdiv)) * Bp + b0;
                    }
                }
            }
            float* go = g_out != nullptr ? g_out + f * Bp + b0 : nullptr;
            uint8_t* ao = addr_out != nullptr ? addr_out + f * Bp + b0 : nullptr;
            // zero the 64 x 32 histogram: 16 conflict-free 16-byte stores per lane
#pragma unroll
            for (int it = 0; it < 16; ++it)
                *reinterpret_cast<float4*>(hist + (it * 32 + lane) * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            __syncwarp();
#define DL_FUSED_ARGS(extra_) valid_chunks, n, extra_, src_lane, sh, gscale_up, words, gdir, ap, gp, tv_r, lowm_r, \
                              inv_ent, e0 + FUSED_MAX_REG_CONTRIB, addr_up, g_up, efd_up, n_up, ugdiv, Bp, b0, go, ao, mine
            if (valid_chunks == FUSED_CG) {
                if (DIRECT) {
                    fused_chunks<true, 0, NIN, true, SWZ, OUTS>(DL_FUSED_ARGS(0));
                } else {
                    switch (cnt) {  // uniform over the warp
                        case 0: fused_chunks<false, 0, NIN, true, SWZ, OUTS>(DL_FUSED_ARGS(0)); break;
                        case 1: fused_chunks<false, 1, NIN, true, SWZ, OUTS>(DL_FUSED_ARGS(0)); break;
                        case 2: fused_chunks<false, 2, NIN, true, SWZ, OUTS>(DL_FUSED_ARGS(0)); break;
                        case 3: fused_chunks<false, 3, NIN, true, SWZ, OUTS>(DL_FUSED_ARGS(0)); break;
                        default:
                            fused_chunks<false, 4, NIN, true, SWZ, OUTS>(DL_FUSED_ARGS(cnt - FUSED_MAX_REG_CONTRIB));
                            break;
                    }
                }
            } else if (DIRECT) {
                fused_chunks<true, 0, NIN, false, SWZ, -1>(DL_FUSED_ARGS(0));
            } else {
                // ragged last group: one generic body, every reader walked through the inverse map
                fused_chunks<false, 5, NIN, false, SWZ, -1>(valid_chunks, n, cnt, src_lane, sh, gscale_up, words, gdir,
                                                            ap, gp, tv_r, lowm_r, inv_ent, e0, addr_up, g_up, efd_up,
                                                            n_up, ugdiv, Bp, b0, go, ao, mine);
            }
#undef DL_FUSED_ARGS
            __syncwarp();
            // group_stride == 0: all groups share one slab.  A node is owned by the same warp in every
            // group and the groups are walked in order, so adding to what this warp stored for the previous
            // group is race-free and sums in group order (the order dl_sum_groups uses).  The previous
            // value is fetched before the reduction below so that its latency hides behind it.
            float* dst = gt_partial + cg * group_stride + f * L;
            float p0 = 0.f, p1 = 0.f;
            if (group_stride == 0 && cg > 0) {
                if (lane < L) p0 = dst[lane];
                if (lane + 32 < L) p1 = dst[lane + 32];
            }
            // sum the 32 lane copies of bins `lane` and `lane + 32`: rotated 16-byte reads, conflict-free
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int col = ((r + lane) & 7) * 4;
                const float4 u = *reinterpret_cast<const float4*>(hist + lane * 32 + col);
                const float4 v = *reinterpret_cast<const float4*>(hist + (lane + 32) * 32 + col);
                s0 += (u.x + u.y) + (u.z + u.w);
                s1 += (v.x + v.y) + (v.z + v.w);
            }
            s0 += p0;
            s1 += p1;
            if (lane < L) dst[lane] = s0;
            if (lane + 32 < L) dst[lane + 32] = s1;
            __syncwarp();
        }
    }
}

// out[i] = sum over groups g (in order) of partial[g*stride + i]
__global__ void sum_groups_kernel(const float* __restrict__ partial, float* __restrict__ out, int64_t count,
                                  int64_t stride, int G) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int g = 0; g < G; ++g) acc += partial[(int64_t)g * stride + i];
        out[i] = acc;
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

// ------------------------------------------------------------------------------------------
// built-in scratch for the entry point that must not allocate
// ------------------------------------------------------------------------------------------

// 16 MiB of device memory owned by the library itself (every GPU that loads it holds this until the
// process exits).  Host code never uses the symbol as a pointer: `static_scratch_address` asks the
// runtime for the symbol's device address once per device and caches it.
constexpr int64_t STATIC_SCRATCH_FLOATS = DL_STATIC_SCRATCH_BYTES / 4;
static __device__ __align__(256) float dl_static_scratch[STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
std::mutex g_scratch_mutex;
float* g_scratch_address[MAX_DEVICES] = {nullptr};

// Device address of dl_static_scratch on the CURRENT device (looked up on first use per device).
int static_scratch_address(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return DL_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_address[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, dl_static_scratch) != cudaSuccess || p == nullptr) return DL_ERR_LAUNCH;
        g_scratch_address[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_address[dev];
    return DL_OK;
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
    DL_REQUIRE(N < ((int64_t)1 << 30));
    const int blocks = grid_for(N * 32, 256);
    if (n == 6)
        dwn_prepare_kernel<6><<<blocks, 256, 0, dl_cast(stream)>>>(tables, efd_t, masks, (int)N, 6, alpha, beta);
    else
        dwn_prepare_kernel<0><<<blocks, 256, 0, dl_cast(stream)>>>(tables, efd_t, masks, (int)N, (int)n, alpha, beta);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_prepare_weighted(const float* tables, float* efd_t, uint64_t* masks, int64_t N, int64_t n,
                                      float scale, const float* hamming_weights_host, dl_stream_t stream) {
    DL_REQUIRE(tables && N > 0 && (efd_t || masks) && hamming_weights_host);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    DL_REQUIRE(N < ((int64_t)1 << 30));
    HammingWeights hw;
    for (int h = 0; h < DL_MAX_FAST_N; ++h) hw.w[h] = h < n ? hamming_weights_host[h] : 0.f;
    const int blocks = (int)dl_min64(N, (int64_t)DL_NUM_SMS * 16);
    dwn_prepare_weighted_kernel<<<blocks, 192, 0, dl_cast(stream)>>>(tables, efd_t, masks, (int)N, (int)n, scale, hw);
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

// Resident CTAs per SM of the persistent bit-sliced forward kernel.  DIFFLUT_FWD_STREAM=0 keeps the layer on the
// one-item-per-thread kernel, =2 / =3 pick the build (measurement aids).
static int fwd_stream_ctas() {
    static const int ctas = [] {
        const char* e = getenv("DIFFLUT_FWD_STREAM");
        if (e && e[0] == '0') return 0;
        if (e && e[0] == '3') return 3;
        return 2;
    }();
    return ctas;
}

DL_EXPORT int dl_dwn_fwd_bits_t(const uint32_t* in_bits_t, const int32_t* map, const uint64_t* masks,
                                uint32_t* out_bits_t, int64_t N, int64_t n, int64_t Bp,
                                dl_stream_t stream) {
    DL_REQUIRE(in_bits_t && map && masks && out_bits_t && N > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(in_bits_t, 16);
    DL_REQUIRE_ALIGNED(out_bits_t, 16);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    DL_REQUIRE(N < ((int64_t)1 << 30) && Bp < ((int64_t)1 << 36));
    const int Q = (int)(Bp / 128);
    int bx = 1;
    while (bx < Q && bx < 256) bx <<= 1;
    const int by = 256 / bx;
    dim3 block(bx, by);
    int64_t gq = dl_ceil_div(Q, bx), gn = dl_ceil_div(N, by);
    if (gq > 65535) gq = 65535;
    const int64_t cap = (int64_t)DL_NUM_SMS * 64;
    if (gn > cap) gn = cap;
    dim3 grid((unsigned)gn, (unsigned)gq);
    cudaStream_t s = dl_cast(stream);
    const int Ni = (int)N;
    if (n == 6 && Q % 32 == 0 && (int64_t)(Q / 32) * N < ((int64_t)1 << 31) && fwd_stream_ctas() > 0) {
        // whole 4096-sample tiles: the persistent, software-pipelined kernel
        const int64_t items = (int64_t)(Q / 32) * N;
        const int ctas = fwd_stream_ctas();
        const int64_t blocks = dl_min64(dl_ceil_div(items, FWD_STREAM_WARPS), (int64_t)DL_NUM_SMS * ctas);
        if (ctas == 3)
            dwn_fwd_bits_stream_kernel<6, 3><<<(unsigned)blocks, FWD_STREAM_WARPS * 32, 0, s>>>(in_bits_t, map, masks,
                                                                                              out_bits_t, Ni, Q);
        else
            dwn_fwd_bits_stream_kernel<6, 2><<<(unsigned)blocks, FWD_STREAM_WARPS * 32, 0, s>>>(in_bits_t, map, masks,
                                                                                              out_bits_t, Ni, Q);
        return dl_launch_status();
    }
#define DL_FWD_BITS(NN)                                                                                      \
    do {                                                                                                     \
        if (bx >= 32)                                                                                        \
            dwn_fwd_bits_kernel<NN, true><<<grid, block, 0, s>>>(in_bits_t, map, masks, out_bits_t, Ni, Q);  \
        else                                                                                                 \
            dwn_fwd_bits_kernel<NN, false><<<grid, block, 0, s>>>(in_bits_t, map, masks, out_bits_t, Ni, Q); \
    } while (0)
    switch (n) {
        case 1: DL_FWD_BITS(1); break;
        case 2: DL_FWD_BITS(2); break;
        case 3: DL_FWD_BITS(3); break;
        case 4: DL_FWD_BITS(4); break;
        case 5: DL_FWD_BITS(5); break;
        default: DL_FWD_BITS(6); break;
    }
#undef DL_FWD_BITS
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_fwd_vals_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                                float* out_t, uint8_t* addr_t, int64_t N, int64_t n, int64_t Bp,
                                dl_stream_t stream) {
    DL_REQUIRE(in_bits_t && map && tables && out_t && N > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(out_t, 16);
    if (addr_t) DL_REQUIRE_ALIGNED(addr_t, 4);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int blocks = grid_for(N * dl_ceil_div(Bp, 1024) * 32, 256);
    dwn_fwd_vals_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(in_bits_t, map, tables, out_t, addr_t, N,
                                                            (int)n, Bp);
    return dl_launch_status();
}

DL_EXPORT int64_t dl_dwn_groupsum_splits(int64_t N, int64_t k) {
    if (N <= 0 || k <= 0) return 1;
    const int64_t gsz = dl_ceil_div(N, k);
    int64_t s = gsz / 8;  // about 8 nodes per slice: enough warps even for one 1024-sample group
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    return s;
}

// Slices per class that a call really uses (<= dl_dwn_groupsum_splits, which sizes the caller's buffer): with
// several 1024-sample groups fewer slices fill the GPU, and every slice costs a cross-warp reduction, 4 KB of
// partial sums per group and one more term in the reduction pass.  DIFFLUT_GROUPSUM_SLICES fixes the count
// (a measurement aid).
static int groupsum_slices_used(int64_t N, int64_t k, int64_t Bp) {
    static const int forced = [] {
        const char* e = getenv("DIFFLUT_GROUPSUM_SLICES");
        return e ? atoi(e) : 0;
    }();
    const int64_t cap = dl_dwn_groupsum_splits(N, k);
    const int64_t groups = dl_ceil_div(Bp, 1024);
    int64_t s = forced > 0 ? forced : dl_ceil_div((int64_t)DL_NUM_SMS * 16, groups * k);
    if (s < 1) s = 1;
    if (s > cap) s = cap;
    return (int)s;
}

// the six-input build of the kernel when it applies, else the one that reads n at run time
#define DL_GROUPSUM_LAUNCH(SWZ) (n == 6 ? dwn_fwd_groupsum_kernel<SWZ, 6> : dwn_fwd_groupsum_kernel<SWZ, 0>)

static int fwd_groupsum_entry(bool swz, const uint32_t* in_bits, const int32_t* map, const float* tables,
                             float* partial, float* logits_t, int64_t N, int64_t n, int64_t k, float tau,
                             int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(in_bits && map && tables && partial && logits_t && N > 0 && k > 0 && tau > 0.f);
    DL_REQUIRE(Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(partial, 16);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int S = groupsum_slices_used(N, k, Bp);
    const int64_t gsz = dl_ceil_div(N, k);
    DL_REQUIRE(k * S <= 65535);
    dim3 grid((unsigned)dl_ceil_div(Bp, 1024), (unsigned)(k * S));
    if (swz)
        DL_GROUPSUM_LAUNCH(true)<<<grid, 128, 0, dl_cast(stream)>>>(in_bits, map, tables, partial, N, (int)n, gsz,
                                                                        S, Bp, dl_swizzled_words(Bp));
    else
        DL_GROUPSUM_LAUNCH(false)<<<grid, 128, 0, dl_cast(stream)>>>(in_bits, map, tables, partial, N, (int)n,
                                                                         gsz, S, Bp, Bp / 32);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    groupsum_reduce_kernel<<<grid_for(k * Bp, 256), 256, 0, dl_cast(stream)>>>(partial, logits_t, (int)k, S,
                                                                            1.0f / tau, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_fwd_groupsum_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                                    float* partial, float* logits_t, int64_t N, int64_t n, int64_t k,
                                    float tau, int64_t Bp, dl_stream_t stream) {
    return fwd_groupsum_entry(false, in_bits_t, map, tables, partial, logits_t, N, n, k, tau, Bp, stream);
}

DL_EXPORT int dl_dwn_fwd_groupsum_s(const uint32_t* in_bits_s, const int32_t* map, const float* tables,
                                    float* partial, float* logits_t, int64_t N, int64_t n, int64_t k,
                                    float tau, int64_t Bp, dl_stream_t stream) {
    return fwd_groupsum_entry(true, in_bits_s, map, tables, partial, logits_t, N, n, k, tau, Bp, stream);
}

DL_EXPORT int dl_dwn_fwd_groupsum_ce_s(const uint32_t* in_bits_s, const int32_t* map, const float* tables,
                                       float* partial, float* logits_t, const int32_t* labels, float* dlogits_t,
                                       float* loss_rows, int64_t N, int64_t n, int64_t k, float tau, int64_t B,
                                       int64_t B_global, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(in_bits_s && map && tables && partial && logits_t && labels && dlogits_t && loss_rows);
    DL_REQUIRE(N > 0 && k > 0 && tau > 0.f && B > 0 && B_global >= B && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(partial, 16);
    if (n < 1 || n > DL_MAX_FAST_N || k > CE_MAX_CLASSES) return DL_ERR_UNSUPPORTED;
    const int S = groupsum_slices_used(N, k, Bp);
    const int64_t gsz = dl_ceil_div(N, k);
    DL_REQUIRE(k * S <= 65535);
    dim3 grid((unsigned)dl_ceil_div(Bp, 1024), (unsigned)(k * S));
    DL_GROUPSUM_LAUNCH(true)<<<grid, 128, 0, dl_cast(stream)>>>(in_bits_s, map, tables, partial, N, (int)n, gsz, S,
                                                                    Bp, dl_swizzled_words(Bp));
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    const int64_t blocks = dl_min64(Bp / 32, (int64_t)DL_NUM_SMS * 8);
    groupsum_reduce_ce_kernel<<<(unsigned)blocks, 256, (size_t)k * 32 * sizeof(float), dl_cast(stream)>>>(
        partial, logits_t, labels, dlogits_t, loss_rows, (int)k, S, 1.0f / tau, B, (float)(1.0 / (double)B_global), Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_fwd_groupsum_noalloc_t(const uint32_t* in_bits_t, const int32_t* map, const float* tables,
                                            float* logits_t, int64_t N, int64_t n, int64_t k, float tau, int64_t Bp,
                                            dl_stream_t stream) {
    DL_REQUIRE(N > 0 && k > 0 && Bp > 0);
    const int64_t need = k * dl_dwn_groupsum_splits(N, k) * Bp;
    if (need > STATIC_SCRATCH_FLOATS) return DL_ERR_TOO_LARGE;
    float* scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc != DL_OK) return rc;
    // every partial sum the reduction pass reads is written by the first pass of this same call, so
    // what an earlier call left in the scratch does not matter and nothing needs clearing
    return dl_dwn_fwd_groupsum_t(in_bits_t, map, tables, scratch, logits_t, N, n, k, tau, Bp, stream);
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
    // chunks per pass: one slab, or as many slabs as it takes to give every resident warp an item (a slab is
    // two items per feature)
    const int64_t resident_warps = (int64_t)DL_NUM_SMS * 5 * 8;
    int64_t slabs = dl_ceil_div(resident_warps, F * 2);
    const int64_t all_slabs = dl_ceil_div(Bp / 128, 8);
    if (slabs > all_slabs) slabs = all_slabs;
    const int cps = (int)(8 * slabs);
    const int64_t want = dl_ceil_div(F * (cps / 4) * 32, 256);  // one warp per (feature, 4 chunks)
    const int blocks = (int)(want < (int64_t)DL_NUM_SMS * 5 ? want : (int64_t)DL_NUM_SMS * 5);
    dwn_bwd_input_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(addr_t, g_t, gdiv, gscale, efd_t, inv_ptr,
                                                             inv_ent, gx_t, F, (int)n, Bp, cps);
    return dl_launch_status();
}

DL_EXPORT int dl_dwn_bwd_input_disjoint_t(const uint8_t* addr_t, const float* g_t, int64_t gdiv, float gscale,
                                          const float* efd_t, const int32_t* map, void* gx_t, int64_t out_bf16,
                                          int64_t NO, int64_t n, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(addr_t && g_t && efd_t && map && gx_t && NO > 0 && gdiv > 0 && gdiv < ((int64_t)1 << 31));
    DL_REQUIRE(Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE_ALIGNED(addr_t, 4);
    DL_REQUIRE_ALIGNED(g_t, 16);
    DL_REQUIRE_ALIGNED(gx_t, 16);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const int64_t items = NO * dl_ceil_div(Bp / 128, 8);
    const int64_t blocks = dl_min64(dl_ceil_div(items, 8), (int64_t)DL_NUM_SMS * 32);
    if (out_bf16)
        dwn_bwd_input_disjoint_kernel<true><<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(
            addr_t, g_t, (uint32_t)gdiv, gscale, efd_t, map, gx_t, NO, (int)n, Bp);
    else
        dwn_bwd_input_disjoint_kernel<false><<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(
            addr_t, g_t, (uint32_t)gdiv, gscale, efd_t, map, gx_t, NO, (int)n, Bp);
    return dl_launch_status();
}

DL_EXPORT int64_t dl_dwn_bwd_groups(int64_t Bp) {
    return Bp <= 0 ? 0 : dl_ceil_div(Bp / 128, FUSED_CG);
}

namespace {

template <bool D, int NN, bool SWZ>
void launch_fused_outs(dim3 grid, cudaStream_t s, const uint8_t* addr_up, const float* g_up, int64_t gdiv_up,
                       float gscale_up, const float* efd_up, int n_up, const int32_t* inv_ptr, const int32_t* inv_ent,
                       const uint32_t* in_bits, const int32_t* map, float* g_out, uint8_t* addr_out, float* gt_partial,
                       int64_t group_stride, int64_t N, int n, int64_t Bp, int64_t Wp) {
#define DL_LAUNCH_FUSED(OUTS)                                                                                         \
    do {                                                                                                              \
        /* enough shared memory for 5 CTAs (5 x 33 KB), the rest stays L1 for index and transform rows */            \
        cudaFuncSetAttribute(dwn_bwd_fused_kernel<D, NN, SWZ, OUTS>, cudaFuncAttributePreferredSharedMemoryCarveout,  \
                              75);                                                                                    \
        dwn_bwd_fused_kernel<D, NN, SWZ, OUTS><<<grid, HIST_WARPS * 32, 0, s>>>(                                       \
            addr_up, g_up, gdiv_up, gscale_up, efd_up, n_up, inv_ptr, inv_ent, in_bits, map, g_out, addr_out,         \
            gt_partial, group_stride, N, n, Bp, Wp);                                                                  \
    } while (0)
    if (NN == 0) {  // generic input count: pointers checked at run time
        DL_LAUNCH_FUSED(-1);
        return;
    }
    switch ((g_out ? 1 : 0) | (addr_out ? 2 : 0)) {
        case 0: DL_LAUNCH_FUSED(0); break;
        case 1: DL_LAUNCH_FUSED(1); break;
        case 2: DL_LAUNCH_FUSED(2); break;
        default: DL_LAUNCH_FUSED(3); break;
    }
#undef DL_LAUNCH_FUSED
}

// Tuning switches read once from the environment (measurement aids; the defaults are the product):
// DIFFLUT_BWD_GENERAL=1 keeps every call on the general kernel, DIFFLUT_BWD_BLOCKS_PER_ITEM=k fixes the
// number of 1024-sample blocks one (node, group) item of the pipelined kernel spans.
struct FusedTuning {
    bool general_only;
    int blocks_per_item;
};
const FusedTuning& fused_tuning() {
    static const FusedTuning t = [] {
        FusedTuning v{false, 0};
        if (const char* e = getenv("DIFFLUT_BWD_GENERAL")) v.general_only = e[0] == '1';
        if (const char* e = getenv("DIFFLUT_BWD_BLOCKS_PER_ITEM")) v.blocks_per_item = atoi(e);
        return v;
    }();
    return t;
}

int bwd_fused_entry(bool swz, const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                    const float* efd_up, int64_t n_up, int64_t N_up, const int32_t* inv_ptr, const int32_t* inv_ent,
                    const uint32_t* in_bits_t, const int32_t* map, float* g_out, uint8_t* addr_out, float* gt_partial,
                    int64_t group_stride, int64_t N, int64_t n, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(g_up && in_bits_t && map && gt_partial && N > 0 && gdiv_up > 0);
    DL_REQUIRE(Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE(group_stride == 0 || group_stride >= N * ((int64_t)1 << n));
    DL_REQUIRE_ALIGNED(g_up, 16);
    if (g_out) DL_REQUIRE_ALIGNED(g_out, 16);
    if (addr_out) DL_REQUIRE_ALIGNED(addr_out, 4);
    if (n < 1 || n > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    const bool direct = (inv_ptr == nullptr);
    if (!direct) {
        DL_REQUIRE(addr_up && efd_up && inv_ent && N_up > 0);
        DL_REQUIRE_ALIGNED(addr_up, 4);
        if (n_up < 1 || n_up > DL_MAX_FAST_N) return DL_ERR_UNSUPPORTED;
    }
    DL_REQUIRE(N < ((int64_t)1 << 28) && gdiv_up < ((int64_t)1 << 31));
    // persistent grid: only as many CTAs as are resident at once, so that the
    // grid-stride loops really sweep all nodes of one 1024-sample slab before the next slab
    // (5 per SM: the register budget of the software-pipelined loads)
    const int64_t cap = (int64_t)DL_NUM_SMS * 5;
    const int64_t blocks64 = dl_ceil_div(N, HIST_WARPS);
    const unsigned blocks = (unsigned)(blocks64 < cap ? blocks64 : cap);
    // few nodes and one slab per group: fill the machine with groups in the grid's second dimension
    int64_t gy = 1;
    if (group_stride > 0 && blocks64 < cap) {
        gy = cap / blocks64;
        const int64_t G = dl_dwn_bwd_groups(Bp);
        if (gy > G) gy = G;
        if (gy < 1) gy = 1;
    }
    const dim3 grid(blocks, (unsigned)gy);
    const int64_t Wp = swz ? dl_swizzled_words(Bp) : Bp / 32;
    cudaStream_t s = dl_cast(stream);
    // the common case (n = 6, interleaved bits, whole 1024-sample blocks) has a software-pipelined kernel
    if (swz && n == 6 && Bp % 1024 == 0 && Bp < ((int64_t)1 << 31) && !fused_tuning().general_only) {
        int bpi = fused_tuning().blocks_per_item;
        if (bpi <= 0) {
            // two blocks per item halve the histogram clear/reduce work; only while every warp slot of the
            // persistent grid still gets several items per launch
            const int64_t items2 = N * (Bp / 2048);
            bpi = (group_stride == 0 && Bp % 2048 == 0 && items2 >= cap * HIST_WARPS * 4) ? 2 : 1;
        }
        const int rc = dl_launch_bwd_pipelined(addr_up, g_up, gdiv_up, gscale_up, efd_up, (int)n_up, inv_ptr, inv_ent,
                                               in_bits_t, map, g_out, addr_out, gt_partial, group_stride, N,
                                               direct ? 0 : N_up, Bp, Wp, bpi, s);
        if (rc != DL_ERR_UNSUPPORTED) return rc;  // else: row offsets beyond 32 bits, general kernel below
    }
#define DL_FUSED_CALL(D, NN, SWZ)                                                                                     \
    launch_fused_outs<D, NN, SWZ>(grid, s, addr_up, g_up, gdiv_up, gscale_up, efd_up, (int)n_up, inv_ptr, inv_ent,  \
                                  in_bits_t, map, g_out, addr_out, gt_partial, group_stride, N, (int)n, Bp, Wp)
    if (swz) {
        if (direct) { if (n == 6) DL_FUSED_CALL(true, 6, true); else DL_FUSED_CALL(true, 0, true); }
        else { if (n == 6) DL_FUSED_CALL(false, 6, true); else DL_FUSED_CALL(false, 0, true); }
    } else {
        if (direct) { if (n == 6) DL_FUSED_CALL(true, 6, false); else DL_FUSED_CALL(true, 0, false); }
        else { if (n == 6) DL_FUSED_CALL(false, 6, false); else DL_FUSED_CALL(false, 0, false); }
    }
#undef DL_FUSED_CALL
    return dl_launch_status();
}

}  // namespace

DL_EXPORT int dl_dwn_bwd_fused_t(const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                                 const float* efd_up, int64_t n_up, int64_t N_up, const int32_t* inv_ptr,
                                 const int32_t* inv_ent, const uint32_t* in_bits_t, const int32_t* map,
                                 float* g_out, uint8_t* addr_out, float* gt_partial, int64_t group_stride,
                                 int64_t N, int64_t n, int64_t Bp, dl_stream_t stream) {
    return bwd_fused_entry(false, addr_up, g_up, gdiv_up, gscale_up, efd_up, n_up, N_up, inv_ptr, inv_ent, in_bits_t, map,
                           g_out, addr_out, gt_partial, group_stride, N, n, Bp, stream);
}

DL_EXPORT int dl_dwn_bwd_fused_s(const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                                 const float* efd_up, int64_t n_up, int64_t N_up, const int32_t* inv_ptr,
                                 const int32_t* inv_ent, const uint32_t* in_bits_s, const int32_t* map,
                                 float* g_out, uint8_t* addr_out, float* gt_partial, int64_t group_stride,
                                 int64_t N, int64_t n, int64_t Bp, dl_stream_t stream) {
    return bwd_fused_entry(true, addr_up, g_up, gdiv_up, gscale_up, efd_up, n_up, N_up, inv_ptr, inv_ent, in_bits_s, map,
                           g_out, addr_out, gt_partial, group_stride, N, n, Bp, stream);
}

DL_EXPORT int dl_sum_groups(const float* partial, float* out, int64_t count, int64_t stride, int64_t groups,
                            dl_stream_t stream) {
    DL_REQUIRE(partial && out && count > 0 && stride >= count && groups > 0);
    sum_groups_kernel<<<grid_for(count, 256), 256, 0, dl_cast(stream)>>>(partial, out, count, stride, (int)groups);
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
