// Fused backward of one DWN layer, n = 6, chunk-interleaved input bits, whole 1024-sample blocks:
// the software-pipelined form of dwn_bwd_fused_kernel (dwn.cu), which stays the general fallback.
//
// What limits this kernel is the SM's load/store data pipe (shuffles, shared-memory and global
// accesses all pass through it, one 128-byte wavefront per cycle), then the latency of the dependent
// loads at the start of every (node, sample group) item.  Three changes against the general kernel:
//
//  * An item may span several 1024-sample blocks (`bpi`): the lane-private histogram is cleared and
//    reduced once per item instead of once per block (128 of the ~450 wavefronts of a one-block item),
//    and it is cleared by the reduction itself (each 16-byte piece is overwritten with zeros right
//    after it is read).
//  * The index data of the NEXT item travels while the current item is computed: its map row and
//    inverse-map bounds are loaded one item ahead (one value per lane, handed out by shuffles), its
//    inverse-map entries at the start of the item's last block, and its input words, EFD values and first two
//    chunks of gradients/addresses are requested before the current item's histogram is reduced.  An item
//    start therefore waits for one memory round trip (overlapped with the reduction) instead of four.
//  * Inside a block the gradients/addresses of chunk c + 2 are requested as soon as chunk c's have been
//    used (reader by reader, into the registers just freed): two chunks are in flight with two buffers,
//    which is what a load that misses L2 needs.
//
// The arithmetic and its order are those of dwn_bwd_fused_kernel: with bpi = 1 both kernels give the
// same bits.  Reference semantics: EFDFunctionCPU.backward, difflut/nodes/dwn_node.py:167-229.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int PW = 4;         // warps per CTA
constexpr int MAXR = 3;       // inverse-map entries of a node kept in registers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}

struct Chunk {            // what one 128-sample chunk needs from the layer above
    uint32_t a[MAXR];     // addresses of the reading nodes (4 samples, one per byte)
    float4 g[MAXR];       // their output gradients (DIRECT: g[0] = this node's own gradient row)
};

// Rows of the layer above are addressed as base + 32-bit element offset (the launcher checks that every
// row offset fits): `oa` into the address bytes, `og` into the gradient floats.  With one gradient row
// per reading node (GSAME) both offsets are the same number and share a register.
template <bool DIRECT, bool GSAME>
__device__ __forceinline__ void load_chunk(Chunk& d, int c, const uint8_t* __restrict__ addr_up,
                                           const float* __restrict__ g_up, const uint32_t (&oa)[MAXR],
                                           const uint32_t (&og)[MAXR]) {
    if (DIRECT) {
        d.g[0] = __ldg(reinterpret_cast<const float4*>(g_up + (size_t)og[0] + c * 128));
    } else {
#pragma unroll
        for (int k = 0; k < MAXR; ++k) {
            d.a[k] = __ldg(reinterpret_cast<const uint32_t*>(addr_up + (size_t)oa[k] + c * 128));
            d.g[k] = __ldg(reinterpret_cast<const float4*>(g_up + (size_t)(GSAME ? oa[k] : og[k]) + c * 128));
        }
    }
}

// one reader's share of a chunk (DIRECT: the node's own gradient row)
template <bool DIRECT, bool GSAME>
__device__ __forceinline__ void load_reader(Chunk& d, int k, int c, const uint8_t* __restrict__ addr_up,
                                            const float* __restrict__ g_up, const uint32_t (&oa)[MAXR],
                                            const uint32_t (&og)[MAXR]) {
    if (DIRECT) {
        d.g[0] = __ldg(reinterpret_cast<const float4*>(g_up + (size_t)og[0] + c * 128));
    } else {
        d.a[k] = __ldg(reinterpret_cast<const uint32_t*>(addr_up + (size_t)oa[k] + c * 128));
        d.g[k] = __ldg(reinterpret_cast<const float4*>(g_up + (size_t)(GSAME ? oa[k] : og[k]) + c * 128));
    }
}

__device__ __forceinline__ void efd_lookup(float4& acc, const float4 g, const uint32_t a, const uint32_t lowm,
                                           const float tv) {
    // lane index of each shuffle = the sample's address without the slot's bit (a shuffle takes its
    // source lane modulo 32, so the bytes above need no masking)
    const uint32_t a5 = (a & lowm) | ((a >> 1) & ~lowm & 0x7F7F7F7Fu);
    acc.x = fmaf(g.x, __shfl_sync(0xffffffffu, tv, a5), acc.x);
    acc.y = fmaf(g.y, __shfl_sync(0xffffffffu, tv, a5 >> 8), acc.y);
    acc.z = fmaf(g.z, __shfl_sync(0xffffffffu, tv, a5 >> 16), acc.z);
    acc.w = fmaf(g.w, __shfl_sync(0xffffffffu, tv, a5 >> 24), acc.w);
}

// One histogram update: bin = byte R of `a`, at shared address mine + bin * 128.
template <int R>
__device__ __forceinline__ void hist_add(uint32_t mine, uint32_t a, float v) {
    const uint32_t bin = __byte_perm(a, 0u, 0x4440u + R);
    const uint32_t at = bin * 128u + mine;
    sts_f32(at, lds_f32(at) + v);
}

template <bool DIRECT, bool GSAME, int OUTS>
__global__ void __launch_bounds__(PW * 32, 5)
dwn_bwd_pipelined_kernel(const uint8_t* __restrict__ addr_up, const float* __restrict__ g_up, uint32_t ugdiv,
                         float gscale, const float* __restrict__ efd_up, int n_up,
                         const int32_t* __restrict__ inv_ptr, const int32_t* __restrict__ inv_ent,
                         const uint32_t* __restrict__ in_bits, const int32_t* __restrict__ map,
                         float* __restrict__ g_out, uint8_t* __restrict__ addr_out, float* __restrict__ gt,
                         int64_t group_stride, int N, uint32_t Bp, uint32_t Wp, int NB, int bpi) {
    __shared__ __align__(16) float hist_all[PW][64 * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* hist = hist_all[warp];                  // hist[e * 32 + lane]: bin e, private to the lane
    const uint32_t mine = smem_u32(hist + lane);
    const int G = (NB + bpi - 1) / bpi;            // items per node
    const int nwarps = gridDim.x * PW;
    const int f0 = blockIdx.x * PW + warp;

#pragma unroll
    for (int it = 0; it < 16; ++it)
        *reinterpret_cast<float4*>(hist + (it * 32 + lane) * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncwarp();

    int cg = blockIdx.y, f = f0;
    if (cg >= G || f >= N) return;

    // index data of one node, one value per lane: lanes 0..5 its map row (input features), lanes 6, 7 the
    // bounds of its inverse-map entries (the readers in the layer above)
    auto load_meta1 = [&](int node) -> int {
        int v = 0;
        if (lane < 6) v = __ldg(map + (int64_t)node * 6 + lane);
        else if (!DIRECT && lane < 8) v = __ldg(inv_ptr + node + (lane - 6));
        return v;
    };
    // the first MAXR inverse-map entries, lanes 0..MAXR-1
    auto load_meta2 = [&](int m1) -> int {
        if (DIRECT) return 0;
        const int e0 = __shfl_sync(0xffffffffu, m1, 6), e1 = __shfl_sync(0xffffffffu, m1, 7);
        int v = 0;
        if (lane < MAXR && lane < e1 - e0) v = __ldg(inv_ent + e0 + lane);
        return v;
    };

    // ---- state of the current item
    uint32_t words[6];
    float tv[MAXR];
    uint32_t lowm[MAXR];
    uint32_t oa[MAXR], og[MAXR];   // element offsets of the readers' rows at this lane's first sample
    uint32_t oo = 0;               // the same for this node's own output rows
    int extra = 0;                 // readers beyond MAXR: walked through the inverse map per chunk
    Chunk even, odd;

    // everything an item needs before its first chunk can be consumed; issues the loads of block
    // `blk0`'s words, the readers' EFD values and chunk 0
    auto setup = [&](int node, int group, int m1, int m2) {
        const uint32_t blk0 = (uint32_t)(group * bpi);
        const uint32_t b0 = blk0 * 1024u + lane * 4;
#pragma unroll
        for (int i = 0; i < 6; ++i) {
            const uint32_t row = (uint32_t)__shfl_sync(0xffffffffu, m1, i);
            words[i] = __ldg(in_bits + (size_t)row * Wp + blk0 * 32u + lane);
        }
        if (DIRECT) {
            og[0] = (ugdiv == 1 ? (uint32_t)node : (uint32_t)node / ugdiv) * Bp + b0;
        } else {
            const int cnt = __shfl_sync(0xffffffffu, m1, 7) - __shfl_sync(0xffffffffu, m1, 6);
            extra = cnt > MAXR ? cnt - MAXR : 0;
#pragma unroll
            for (int k = 0; k < MAXR; ++k) {
                const uint32_t ent = (uint32_t)__shfl_sync(0xffffffffu, m2, k);
                const uint32_t j = ent >> 3, i = ent & 7u;
                // absent readers keep valid offsets (node 0) and contribute exactly zero
                const float t = __ldg(efd_up + ((size_t)j * n_up + i) * 32 + lane);
                tv[k] = k < cnt ? gscale * t : 0.f;
                lowm[k] = ((1u << i) - 1u) * 0x01010101u;
                oa[k] = j * Bp + b0;
                if (!GSAME) og[k] = (ugdiv == 1 ? j : j / ugdiv) * Bp + b0;
            }
        }
        if (OUTS != 0) oo = (uint32_t)node * Bp + b0;
        load_chunk<DIRECT, GSAME>(even, 0, addr_up, g_up, oa, og);  // chunk 1 follows once the caller has registers for it
    };

    // the next 1024-sample block of the same node
    auto next_block = [&](int m1, int blk) {
#pragma unroll
        for (int i = 0; i < 6; ++i) {
            const uint32_t row = (uint32_t)__shfl_sync(0xffffffffu, m1, i);
            words[i] = __ldg(in_bits + (size_t)row * Wp + (uint32_t)blk * 32u + lane);
        }
        if (DIRECT) {
            og[0] += 1024u;
        } else {
#pragma unroll
            for (int k = 0; k < MAXR; ++k) {
                oa[k] += 1024u;
                if (!GSAME) og[k] += 1024u;
            }
        }
        if (OUTS != 0) oo += 1024u;
        load_chunk<DIRECT, GSAME>(even, 0, addr_up, g_up, oa, og);
        load_chunk<DIRECT, GSAME>(odd, 1, addr_up, g_up, oa, og);
    };

    // Chunk c of the current block.  As soon as a reader's address word and gradients have been used, the
    // same registers receive that reader's data of chunk c + 2: two chunks are in flight with two buffers.
    // EXTRA: the node has more readers than registers (rare); they are walked through the inverse map.
    auto consume = [&](Chunk& d, int c, int blk, int m1cur, auto extra_tag) {
        constexpr bool EXTRA = decltype(extra_tag)::value;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (DIRECT) {
            acc = d.g[0];
            acc.x *= gscale; acc.y *= gscale; acc.z *= gscale; acc.w *= gscale;
            if (c + 2 < 8) load_reader<DIRECT, GSAME>(d, 0, c + 2, addr_up, g_up, oa, og);
        } else {
#pragma unroll
            for (int k = 0; k < MAXR; ++k) {
                efd_lookup(acc, d.g[k], d.a[k], lowm[k], tv[k]);
                if (c + 2 < 8) load_reader<DIRECT, GSAME>(d, k, c + 2, addr_up, g_up, oa, og);
            }
            if (EXTRA)
            for (int k = 0; k < extra; ++k) {
                const int ent = __ldg(&inv_ent[__shfl_sync(0xffffffffu, m1cur, 6) + MAXR + k]);
                const uint32_t j = (uint32_t)ent >> 3, i = (uint32_t)ent & 7u;
                const float t = gscale * __ldg(efd_up + ((size_t)j * n_up + i) * 32 + lane);
                const uint32_t off = (uint32_t)blk * 1024u + lane * 4 + c * 128;
                const uint32_t a = __ldg(reinterpret_cast<const uint32_t*>(addr_up + (size_t)(j * Bp + off)));
                const float4 g = __ldg(reinterpret_cast<const float4*>(
                    g_up + (size_t)((ugdiv == 1 ? j : j / ugdiv) * Bp + off)));
                efd_lookup(acc, g, a, ((1u << i) - 1u) * 0x01010101u, t);
            }
        }
        // own addresses: bit c + 8r of the lane's word i is input i of its sample r of chunk c
        uint32_t a = 0;
#pragma unroll
        for (int i = 0; i < 6; ++i) {
            const uint32_t t = c >= i ? words[i] >> (c - i) : words[i] << (i - c);
            a |= t & (0x01010101u << i);
        }
        if (OUTS & 1) *reinterpret_cast<float4*>(g_out + (size_t)oo + c * 128) = acc;
        if (OUTS & 2) *reinterpret_cast<uint32_t*>(addr_out + (size_t)oo + c * 128) = a;
        hist_add<0>(mine, a, acc.x);
        hist_add<1>(mine, a, acc.y);
        hist_add<2>(mine, a, acc.z);
        hist_add<3>(mine, a, acc.w);
    };

    // ---- prologue: the first item's index data (the only place where the chain is waited for)
    int m1 = load_meta1(f);
    int ncg = cg, nf = f + nwarps;
    if (nf >= N) { nf = f0; ncg = cg + gridDim.y; }
    bool nvalid = ncg < G;
    int m1n = nvalid ? load_meta1(nf) : 0;
    int m2n = 0;
    {
        const int m2 = load_meta2(m1);
        setup(f, cg, m1, m2);
    }
    load_chunk<DIRECT, GSAME>(odd, 1, addr_up, g_up, oa, og);

    while (true) {
        const int blk_first = cg * bpi;
        const int blk_end = blk_first + bpi < NB ? blk_first + bpi : NB;
        for (int blk = blk_first; blk < blk_end; ++blk) {
            const bool last_blk = blk + 1 == blk_end;
            if (last_blk && nvalid) m2n = load_meta2(m1n);  // uniform over the warp; used at the item's end
            if (extra == 0) {
#pragma unroll
                for (int c = 0; c < 8; c += 2) {
                    consume(even, c, blk, m1, std::false_type{});
                    consume(odd, c + 1, blk, m1, std::false_type{});
                }
            } else {
#pragma unroll
                for (int c = 0; c < 8; c += 2) {
                    consume(even, c, blk, m1, std::true_type{});
                    consume(odd, c + 1, blk, m1, std::true_type{});
                }
            }
            if (!last_blk) next_block(m1, blk + 1);
        }
        // ---- the next item's loads start before this item's histogram is reduced
        float* dst = gt + (int64_t)cg * group_stride + (int64_t)f * 64;
        const bool add_prev = group_stride == 0 && cg > 0;
        const bool more = nvalid;
        if (more) {
            m1 = m1n;
            f = nf;
            cg = ncg;
            setup(f, cg, m1, m2n);
            nf = f + nwarps;
            if (nf >= N) { nf = f0; ncg = cg + gridDim.y; }
            nvalid = ncg < G;
            m1n = nvalid ? load_meta1(nf) : 0;
        }
        __syncwarp();
        // all groups share one slab when group_stride == 0: a node belongs to the same warp in every group and
        // the groups are walked in order, so adding to what this warp stored for the previous group is
        // race-free and sums in group order
        float p0 = 0.f, p1 = 0.f;
        if (add_prev) {
            p0 = dst[lane];
            p1 = dst[lane + 32];
        }
        // sum the 32 lane copies of bins `lane` and `lane + 32` (rotated 16-byte reads, conflict-free) and leave
        // zeros behind for the next item
        float s0 = 0.f, s1 = 0.f;
#pragma unroll 2  // more in flight would collide with the next item's registers, which are already live
        for (int r = 0; r < 8; ++r) {
            const int col = ((r + lane) & 7) * 4;
            float4* pu = reinterpret_cast<float4*>(hist + lane * 32 + col);
            float4* pv = reinterpret_cast<float4*>(hist + (lane + 32) * 32 + col);
            const float4 u = *pu, v = *pv;
            *pu = make_float4(0.f, 0.f, 0.f, 0.f);
            *pv = make_float4(0.f, 0.f, 0.f, 0.f);
            s0 += (u.x + u.y) + (u.z + u.w);
            s1 += (v.x + v.y) + (v.z + v.w);
        }
        s0 += p0;
        s1 += p1;
        dst[lane] = s0;
        dst[lane + 32] = s1;
        __syncwarp();
        if (!more) break;
        load_chunk<DIRECT, GSAME>(odd, 1, addr_up, g_up, oa, og);  // the reduction's registers are free again
    }
}

}  // namespace

// Launches the pipelined kernel, or returns DL_ERR_UNSUPPORTED when a row offset does not fit 32 bits (the
// caller then uses the general kernel).  The caller (bwd_fused_entry in dwn.cu) has validated the arguments
// and checked n == 6, interleaved bits and Bp % 1024 == 0.  blocks_per_item >= 1.
int dl_launch_bwd_pipelined(const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                            const float* efd_up, int n_up, const int32_t* inv_ptr, const int32_t* inv_ent,
                            const uint32_t* in_bits, const int32_t* map, float* g_out, uint8_t* addr_out,
                            float* gt, int64_t group_stride, int64_t N, int64_t N_up, int64_t Bp, int64_t Wp,
                            int blocks_per_item, cudaStream_t s) {
    const int64_t rows = N > N_up ? N : N_up;
    if (rows * Bp >= ((int64_t)1 << 32) || Wp >= ((int64_t)1 << 31)) return DL_ERR_UNSUPPORTED;
    const int NB = (int)(Bp / 1024);
    int bpi = blocks_per_item < 1 ? 1 : blocks_per_item;
    if (group_stride > 0) bpi = 1;  // one slab per 1024-sample group: items cannot span blocks
    if (bpi > NB) bpi = NB;
    const int G = (NB + bpi - 1) / bpi;
    const int64_t cap = (int64_t)DL_NUM_SMS * 5;  // persistent grid: the CTAs resident at once
    const int64_t blocks64 = dl_ceil_div(N, PW);
    const unsigned blocks = (unsigned)(blocks64 < cap ? blocks64 : cap);
    int64_t gy = 1;
    if (group_stride > 0 && blocks64 < cap) {  // few nodes, independent slabs: groups side by side
        gy = cap / blocks64;
        if (gy > G) gy = G;
        if (gy < 1) gy = 1;
    }
    const dim3 grid(blocks, (unsigned)gy);
    const bool direct = inv_ptr == nullptr;
    const bool gsame = gdiv_up == 1;
    const int outs = (g_out ? 1 : 0) | (addr_out ? 2 : 0);
#define DL_PIPE(D, S, O)                                                                                            \
    do {                                                                                                            \
        /* enough shared memory for 5 CTAs (5 x 33 KB), the rest stays L1 for index and transform rows */           \
        cudaFuncSetAttribute(dwn_bwd_pipelined_kernel<D, S, O>, cudaFuncAttributePreferredSharedMemoryCarveout, 75); \
        dwn_bwd_pipelined_kernel<D, S, O><<<grid, PW * 32, 0, s>>>(                                                 \
            addr_up, g_up, (uint32_t)gdiv_up, gscale_up, efd_up, n_up, inv_ptr, inv_ent, in_bits, map, g_out,       \
            addr_out, gt, group_stride, (int)N, (uint32_t)Bp, (uint32_t)Wp, NB, bpi);                               \
    } while (0)
#define DL_PIPE_OUTS(D, S)                    \
    switch (outs) {                           \
        case 0: DL_PIPE(D, S, 0); break;      \
        case 1: DL_PIPE(D, S, 1); break;      \
        case 2: DL_PIPE(D, S, 2); break;      \
        default: DL_PIPE(D, S, 3); break;     \
    }
    if (direct) {
        DL_PIPE_OUTS(true, false)
    } else if (gsame) {
        DL_PIPE_OUTS(false, true)
    } else {
        DL_PIPE_OUTS(false, false)
    }
#undef DL_PIPE_OUTS
#undef DL_PIPE
    return dl_launch_status();
}
