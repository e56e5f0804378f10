// Thermometer encoder and layout-change kernels.
//
// The reference encoder (difflut/encoder/thermometer.py:89-116) writes one fp32 per bit.  The
// kernels here compare once and either write that fp32 tensor (API-exact) or ballot the
// results of 32 samples into one word of the packed feature-major layout the LUT kernels read.
#include "common.cuh"

namespace {

constexpr int TILE_F = 32;    // features per CTA tile
constexpr int TILE_B = 256;   // samples per CTA tile (8 words per feature row)
constexpr int PACK_THREADS = 256;

// x rows (B,F) -> packed feature-major bits.  MODE 0: bit = x > thr[f][t] (T bits per feature);
// MODE 1: bit = x >= scalar threshold (T == 1).  A CTA stages a 256-sample x 32-feature tile in
// shared memory (coalesced row reads), then each warp takes 4 features: for every threshold it
// ballots the 8 words of the tile and lanes 0..7 store them as one 32-byte piece of the output row.
template <int MODE>
__global__ void __launch_bounds__(PACK_THREADS)
pack_t_kernel(const float* __restrict__ x, const float* __restrict__ thr, float scalar_thr,
              uint32_t* __restrict__ bits_t, int64_t B, int64_t F, int T, int64_t Wp) {
    __shared__ float tile[TILE_B][TILE_F + 1];
    const int64_t f0 = (int64_t)blockIdx.y * TILE_F;
    const int64_t b0 = (int64_t)blockIdx.x * TILE_B;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // coalesced load: one warp reads 32 consecutive features of one sample row
#pragma unroll 8
    for (int r = warp; r < TILE_B; r += PACK_THREADS / 32) {
        const int64_t b = b0 + r, f = f0 + lane;
        tile[r][lane] = (b < B && f < F) ? x[b * F + f] : 0.0f;
    }
    __syncthreads();
    const int64_t word0 = b0 >> 5;
    for (int fl = warp * 4; fl < warp * 4 + 4; ++fl) {
        const int64_t f = f0 + fl;
        if (f >= F) break;  // uniform over the warp
        float v[8];
        bool valid[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            v[k] = tile[k * 32 + lane][fl];
            valid[k] = b0 + k * 32 + lane < B;
        }
        for (int t = 0; t < T; ++t) {
            const float th = MODE == 0 ? __ldg(&thr[f * T + t]) : scalar_thr;
            uint32_t mine = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const bool bit = valid[k] && (MODE == 0 ? v[k] > th : v[k] >= th);
                const uint32_t w = __ballot_sync(0xffffffffu, bit);
                if (lane == k) mine = w;
            }
            if (lane < 8 && word0 + lane < Wp) bits_t[(f * T + t) * Wp + word0 + lane] = mine;
        }
    }
}

// Natural feature-major bits -> chunk-interleaved layout used by the stack kernels.  Per 1024-sample
// block a row has 32 words; word w, bit c + 8r holds sample 128c + 4w + r of the block (c = 0..7 the
// 128-sample chunk, r = 0..3).  A warp owns one (row, block): lane w reads natural word w (coalesced),
// then collects nibble (w % 8) of natural word 4c + w/8 for every c and spreads it over the bytes.
__global__ void __launch_bounds__(256)
bits_swizzle_kernel(const uint32_t* __restrict__ nat, uint32_t* __restrict__ swz, int64_t F, int64_t Wp,
                    int64_t G) {
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int src = lane >> 3, sh = (lane & 7) * 4;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < F * G; item += nwarps) {
        const int64_t f = item / G, g = item - f * G;
        const int64_t w = g * 32 + lane;
        const uint32_t mine = w < Wp ? __ldg(nat + f * Wp + w) : 0u;
        uint32_t out = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t t = __shfl_sync(0xffffffffu, mine, c * 4 + src) >> sh;
            out |= dl_spread_nibble(t & 0xFu) << c;
        }
        swz[(f * G + g) * 32 + lane] = out;
    }
}

// Thermometer compare-and-pack straight into the chunk-interleaved layout (see bits_swizzle_kernel).
// A CTA owns one 1024-sample block and FEATS features (one warp per feature).  The block's values go to
// shared memory as tile[feature][q][w] with q = c + 8r the bit position and w the word of sample
// 128c + 4w + r (row pitch 33, feature pitch 1057: fill and read-out are both bank-conflict free).
// Fill: with 16-byte-aligned rows (VEC4) a thread fetches four features of a sample per load and has all
// of its eight loads in flight before the first value is stored; otherwise 4-byte loads.  Lane w of warp k
// then holds the 32 values of word w of feature k in registers, in bit order, and builds each threshold's
// word with two instructions per bit: the sign of (threshold - value) is exactly the strict comparison
// value > threshold for finite thresholds (the difference of two floats is zero only when they are equal,
// and a NaN, which is what padding samples hold, keeps its positive sign), and a funnel shift moves it into
// the word.  The 32 words of a (feature, threshold) row leave as one coalesced 128-byte store.
constexpr int SWZ_ROW = 33, SWZ_FEAT = 32 * SWZ_ROW + 1;

__device__ __forceinline__ int swz_slot(int s) {  // sample s of the block -> q * SWZ_ROW + w
    return (((s >> 7) + 8 * (s & 3)) * SWZ_ROW) + ((s >> 2) & 31);
}

template <int FEATS, bool VEC4>
__global__ void __launch_bounds__(FEATS * 32)
thermo_pack_s_kernel(const float* __restrict__ x, const float* __restrict__ thr, uint32_t* __restrict__ bits_s,
                     int64_t B, int64_t F, int T, int64_t G) {
    __shared__ float tile[FEATS * SWZ_FEAT];
    const int64_t g = blockIdx.x;
    const int64_t f0 = (int64_t)blockIdx.y * FEATS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float nan = __int_as_float(0x7fc00000);  // (threshold - NaN) keeps the positive sign: padding packs as 0
    if (VEC4) {
        constexpr int QUADS = FEATS / 4;               // 16-byte pieces per sample
        constexpr int ROWS = FEATS * 32 / QUADS;       // samples per pass
        constexpr int PASSES = 1024 / ROWS;
        const int h = threadIdx.x % QUADS, s0 = threadIdx.x / QUADS;
        const int64_t f = f0 + 4 * h;
        float4 v[PASSES];
#pragma unroll
        for (int k = 0; k < PASSES; ++k) {
            const int64_t b = g * 1024 + s0 + k * ROWS;
            v[k] = (b < B && f < F) ? __ldg(reinterpret_cast<const float4*>(x + b * F + f)) : make_float4(nan, nan, nan, nan);
        }
#pragma unroll
        for (int k = 0; k < PASSES; ++k) {
            float* dst = tile + (4 * h) * SWZ_FEAT + swz_slot(s0 + k * ROWS);
            dst[0] = v[k].x;
            dst[SWZ_FEAT] = v[k].y;
            dst[2 * SWZ_FEAT] = v[k].z;
            dst[3 * SWZ_FEAT] = v[k].w;
        }
    } else {
        const int fl = threadIdx.x % FEATS;
        for (int s = threadIdx.x / FEATS; s < 1024; s += 32) {
            const int64_t b = g * 1024 + s, f = f0 + fl;
            tile[fl * SWZ_FEAT + swz_slot(s)] = (b < B && f < F) ? __ldg(x + b * F + f) : nan;
        }
    }
    __syncthreads();
    const int64_t f = f0 + warp;
    if (f >= F) return;
    float v[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) v[q] = tile[warp * SWZ_FEAT + q * SWZ_ROW + lane];
    for (int t = 0; t < T; ++t) {
        const float th = __fadd_rn(__ldg(&thr[f * T + t]), 0.0f);  // a threshold of -0 counts as +0
        uint32_t word = 0;
#pragma unroll
        for (int q = 31; q >= 0; --q)  // (word << 1) | sign bit of (th - v[q])
            word = __funnelshift_l(__float_as_uint(__fsub_rn(th, v[q])), word, 1);
        bits_s[((f * T + t) * G + g) * 32 + lane] = word;
    }
}

// Feature-major fp32 [F][ld] (B valid samples per row) -> packed feature-major bits [F][Wp], bit = value >=
// threshold.  A warp takes 128 samples of one row: four coalesced loads, four ballots, lanes 0..3 store.
__global__ void __launch_bounds__(256)
pack_t_to_t_kernel(const float* __restrict__ src_t, uint32_t* __restrict__ bits_t, int64_t F, int64_t B,
                   int64_t ld, int64_t Wp, float threshold) {
    const int lane = threadIdx.x & 31;
    const int64_t Q = Wp >> 2;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < F * Q; item += nwarps) {
        const int64_t f = item / Q, q = item - f * Q;
        const float* row = src_t + f * ld;
        uint32_t mine = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t b = (q * 4 + k) * 32 + lane;
            const bool bit = b < B && __ldg(row + b) >= threshold;
            const uint32_t word = __ballot_sync(0xffffffffu, bit);
            if (lane == k) mine = word;
        }
        if (lane < 4) bits_t[f * Wp + q * 4 + lane] = mine;
    }
}

// The same with 16-byte loads: a warp item is 512 samples of one feature; a lane reads four float4 (one per
// 128-sample chunk, all in flight together), turns each into a nibble, and the eight nibbles of a word are
// combined with a warp OR.  Needs ld % 4 == 0 and a 16-byte aligned source.
__global__ void __launch_bounds__(256)
pack_t_to_t_vec_kernel(const float* __restrict__ src_t, uint32_t* __restrict__ bits_t, int64_t F, int64_t B,
                       int64_t ld, int64_t Wp, float threshold) {
    const int lane = threadIdx.x & 31;
    const int64_t C = Wp >> 2;             // 128-sample chunks per row
    const int64_t Q = (C + 3) >> 2;        // items per row
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t item = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; item < F * Q; item += nwarps) {
        const int64_t f = item / Q, q = item - f * Q;
        const float* row = src_t + f * ld;
        float4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t c = q * 4 + k;
            v[k] = c < C ? __ldg(reinterpret_cast<const float4*>(row + c * 128) + lane)
                         : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t c = q * 4 + k;
            if (c >= C) break;  // uniform over the warp
            const int64_t b = c * 128 + lane * 4;
            uint32_t nib = 0;
            nib |= (b + 0 < B && v[k].x >= threshold) ? 1u : 0u;
            nib |= (b + 1 < B && v[k].y >= threshold) ? 2u : 0u;
            nib |= (b + 2 < B && v[k].z >= threshold) ? 4u : 0u;
            nib |= (b + 3 < B && v[k].w >= threshold) ? 8u : 0u;
            const uint32_t part = nib << ((lane & 7) * 4);
            uint32_t mine = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t word = __reduce_or_sync(0xffffffffu, (lane >> 3) == w ? part : 0u);
                if (lane == w) mine = word;
            }
            if (lane < 4) bits_t[f * Wp + c * 4 + lane] = mine;
        }
    }
}

// rows in, fp32 rows out: out[b, f*T+t] = x[b,f] > thr[f,t]
__global__ void thermo_rows_kernel(const float* __restrict__ x, const float* __restrict__ thr,
                                   float* __restrict__ out, int64_t B, int64_t F, int T) {
    const int64_t total = B * F * T;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = i % (F * T), b = i / (F * T);
        const int64_t f = c / T;
        out[i] = (x[b * F + f] > __ldg(&thr[c])) ? 1.0f : 0.0f;
    }
}

// The same for row lengths F*T that are multiples of 4: a thread owns four adjacent output columns, looks their
// features and thresholds up once, and then walks the samples of its grid row with one 16-byte store each
// (no division inside the loop).
__global__ void __launch_bounds__(256)
thermo_rows_vec_kernel(const float* __restrict__ x, const float* __restrict__ thr, float* __restrict__ out,
                       int64_t B, int64_t F, int T, int C4) {
    const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c4 >= C4) return;
    const int c = c4 * 4;
    const int f0 = c / T, f1 = (c + 1) / T, f2 = (c + 2) / T, f3 = (c + 3) / T;
    const float4 th = __ldg(reinterpret_cast<const float4*>(thr) + c4);
    const int64_t C = (int64_t)C4 * 4;
    for (int64_t b = blockIdx.y; b < B; b += gridDim.y) {
        const float* xr = x + b * F;
        const float v0 = __ldg(xr + f0), v1 = __ldg(xr + f1), v2 = __ldg(xr + f2), v3 = __ldg(xr + f3);
        *reinterpret_cast<float4*>(out + b * C + c) =
            make_float4(v0 > th.x ? 1.0f : 0.0f, v1 > th.y ? 1.0f : 0.0f, v2 > th.z ? 1.0f : 0.0f, v3 > th.w ? 1.0f : 0.0f);
    }
}

// rows in, packed rows out: one warp per (sample, word); lane = column inside the word
__global__ void thermo_pack_rows_kernel(const float* __restrict__ x, const float* __restrict__ thr,
                                        uint32_t* __restrict__ bits, int64_t B, int64_t F, int T,
                                        int64_t Wr) {
    const int64_t C = F * T;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < B * Wr; w += nwarps) {
        const int64_t b = w / Wr, c = (w % Wr) * 32 + lane;
        bool bit = false;
        if (c < C) bit = x[b * F + c / T] > __ldg(&thr[c]);
        const uint32_t word = __ballot_sync(0xffffffffu, bit);
        if (lane == 0) bits[w] = word;
    }
}

// fp32 rows (B,F) -> feature-major [F][Bp] through a 32x32 shared tile; padding written as 0.
__global__ void __launch_bounds__(256)
rows_to_t_kernel(const float* __restrict__ rows, float* __restrict__ t, int64_t B, int64_t F,
                 int64_t Bp) {
    __shared__ float tile[32][33];
    const int64_t f0 = (int64_t)blockIdx.y * 32, b0 = (int64_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t b = b0 + r, f = f0 + tx;
        tile[r][tx] = (b < B && f < F) ? rows[b * F + f] : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int64_t f = f0 + r, b = b0 + tx;
        if (f < F && b < Bp) t[f * Bp + b] = tile[tx][r];
    }
}

__global__ void __launch_bounds__(256)
t_to_rows_kernel(const float* __restrict__ t, float* __restrict__ rows, int64_t B, int64_t F,
                 int64_t Bp) {
    __shared__ float tile[32][33];
    const int64_t f0 = (int64_t)blockIdx.y * 32, b0 = (int64_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t f = f0 + r, b = b0 + tx;
        tile[r][tx] = (f < F && b < Bp) ? t[f * Bp + b] : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int64_t b = b0 + r, f = f0 + tx;
        if (b < B && f < F) rows[b * F + f] = tile[tx][r];
    }
}

// 64 x 64 tiles with 16-byte accesses on both sides, for shapes whose row lengths are multiples of 4 and
// whose pointers are 16-byte aligned: dst[c][r] = src[r][c].  Source rows r >= R read as zero; source columns are
// loaded while c < c_load and stored (as destination rows) while c < C; destination columns are written up to
// r_store.  Twice the bytes in flight per thread of the 32 x 32 form above.
__global__ void __launch_bounds__(256)
transpose64_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t R, int64_t C, int64_t c_load,
                   int64_t r_store, int64_t ld_src, int64_t ld_dst) {
    __shared__ float tile[64][65];
    const int64_t r0 = (int64_t)blockIdx.x * 64, c0 = (int64_t)blockIdx.y * 64;
    const int q = threadIdx.x & 15, p = threadIdx.x >> 4;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = p + 16 * k;
        const int64_t gr = r0 + r, gc = c0 + 4 * q;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gr < R && gc < c_load) v = __ldg(reinterpret_cast<const float4*>(src + gr * ld_src + gc));
        tile[r][4 * q + 0] = v.x;
        tile[r][4 * q + 1] = v.y;
        tile[r][4 * q + 2] = v.z;
        tile[r][4 * q + 3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c = p + 16 * k;
        const int64_t gc = c0 + c, gr = r0 + 4 * q;
        if (gc < C && gr < r_store)
            *reinterpret_cast<float4*>(dst + gc * ld_dst + gr) =
                make_float4(tile[4 * q + 0][c], tile[4 * q + 1][c], tile[4 * q + 2][c], tile[4 * q + 3][c]);
    }
}

static bool transpose64_ok(const void* a, const void* b, int64_t n0, int64_t n1) {
    return reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0 && n0 % 4 == 0 &&
           n1 % 4 == 0;
}

// bits_t [F][Wp] -> fp32 rows (B,F) of {0,1}: CTA tile = 32 features x 32 samples (one word each)
__global__ void __launch_bounds__(256)
bits_t_to_rows_kernel(const uint32_t* __restrict__ bits_t, float* __restrict__ rows, int64_t B,
                      int64_t F, int64_t Wp) {
    __shared__ uint32_t words[32];
    const int64_t f0 = (int64_t)blockIdx.y * 32, w = blockIdx.x;
    if (threadIdx.x < 32) {
        const int64_t f = f0 + threadIdx.x;
        words[threadIdx.x] = f < F ? bits_t[f * Wp + w] : 0u;
    }
    __syncthreads();
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t b = w * 32 + r, f = f0 + tx;
        if (b < B && f < F) rows[b * F + f] = (float)((words[tx] >> r) & 1u);
    }
}

// packed rows (B, Wr) -> packed feature-major [F][Wp].  A CTA takes 512 samples x 8 column words
// (256 features): the 512 x 8 input words are read with 32-byte row pieces into shared memory,
// every warp transposes 32x32 bit tiles with five shuffle rounds, and the 256 x 16 output words leave as 64-byte row pieces.
__global__ void __launch_bounds__(256)
bits_rows_to_t_kernel(const uint32_t* __restrict__ bits_rows, uint32_t* __restrict__ bits_t,
                      int64_t B, int64_t F, int64_t Wr, int64_t Wp) {
    // one buffer for both directions (18 KB: eight CTAs per SM): the input tile [512][9] (+1 word padding: a warp
    // reads one column conflict-free) is overwritten by the output tile [256][17] once every warp holds its words
    __shared__ uint32_t tile_buf[512 * 9];
    uint32_t (*in_tile)[9] = reinterpret_cast<uint32_t (*)[9]>(tile_buf);
    uint32_t (*out_tile)[17] = reinterpret_cast<uint32_t (*)[17]>(tile_buf);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t wc0 = (int64_t)blockIdx.y * 8;      // first column word
    const int64_t b0 = (int64_t)blockIdx.x * 512;     // first sample
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const int idx = threadIdx.x + k * 256;
        const int r = idx >> 3, cw = idx & 7;
        const int64_t b = b0 + r, wc = wc0 + cw;
        in_tile[r][cw] = (b < B && wc < Wr) ? __ldg(bits_rows + b * Wr + wc) : 0u;
    }
    __syncthreads();
    // 8 column words x 16 sample words = 128 tiles; warp w takes column word w
    uint32_t held[16];
#pragma unroll
    for (int sw = 0; sw < 16; ++sw) held[sw] = in_tile[sw * 32 + lane][warp];
    __syncthreads();  // the input tile may be overwritten now
#pragma unroll
    // 32x32 bit transpose across the warp: five rounds of swapping off-diagonal blocks with the lane that
    // differs in bit j of its index (lane r starts with sample r's word and ends with the 32 samples of
    // feature r).  A lane with bit j clear keeps its low halves and takes the partner's low halves shifted up;
    // a lane with bit j set keeps its high halves and takes the partner's high halves shifted down.  For
    // j = 16 and 8 that is one byte permute; for j = 4, 2, 1 one rotate of the partner's word and one
    // three-input select, with the selector / rotate amount / keep mask of each lane prepared once.
    const uint32_t sel16 = (lane & 16) ? 0x3276u : 0x5410u;
    const uint32_t sel8 = (lane & 8) ? 0x3715u : 0x6240u;
    const uint32_t rot4 = (lane & 4) ? 28u : 4u, keep4 = (lane & 4) ? 0xF0F0F0F0u : 0x0F0F0F0Fu;
    const uint32_t rot2 = (lane & 2) ? 30u : 2u, keep2 = (lane & 2) ? 0xCCCCCCCCu : 0x33333333u;
    const uint32_t rot1 = (lane & 1) ? 31u : 1u, keep1 = (lane & 1) ? 0xAAAAAAAAu : 0x55555555u;
#pragma unroll
    for (int sw = 0; sw < 16; ++sw) {
        uint32_t v = held[sw];
        v = __byte_perm(v, __shfl_xor_sync(0xffffffffu, v, 16), sel16);
        v = __byte_perm(v, __shfl_xor_sync(0xffffffffu, v, 8), sel8);
        uint32_t p = __shfl_xor_sync(0xffffffffu, v, 4);
        v = (v & keep4) | (__funnelshift_l(p, p, rot4) & ~keep4);
        p = __shfl_xor_sync(0xffffffffu, v, 2);
        v = (v & keep2) | (__funnelshift_l(p, p, rot2) & ~keep2);
        p = __shfl_xor_sync(0xffffffffu, v, 1);
        v = (v & keep1) | (__funnelshift_l(p, p, rot1) & ~keep1);
        out_tile[warp * 32 + lane][sw] = v;
    }
    __syncthreads();
    const int64_t wb0 = b0 >> 5;
    for (int row = warp; row < 256; row += 8) {
        const int64_t f = wc0 * 32 + row;
        if (lane < 16 && f < F && wb0 + lane < Wp) bits_t[f * Wp + wb0 + lane] = out_tile[row][lane];
    }
}

}  // namespace

DL_EXPORT int dl_thermo_rows(const float* x, const float* thr, float* out, int64_t B, int64_t F,
                             int64_t T, dl_stream_t stream) {
    DL_REQUIRE(x && thr && out && B > 0 && F > 0 && T > 0);
    const int64_t total = B * F * T;
    if ((F * T) % 4 == 0 && F * T < ((int64_t)1 << 31) && reinterpret_cast<uintptr_t>(thr) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(out) % 16 == 0) {
        const int C4 = (int)(F * T / 4);
        const unsigned gx = (unsigned)dl_ceil_div(C4, 256);
        const int64_t gy = dl_min64(B, dl_max64(1, (int64_t)DL_NUM_SMS * 16 / gx));
        thermo_rows_vec_kernel<<<dim3(gx, (unsigned)gy), 256, 0, dl_cast(stream)>>>(x, thr, out, B, F, (int)T, C4);
        return dl_launch_status();
    }
    const int blocks = (int)dl_min64(dl_ceil_div(total, 256), (int64_t)DL_NUM_SMS * 16);
    thermo_rows_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(x, thr, out, B, F, (int)T);
    return dl_launch_status();
}

DL_EXPORT int dl_thermo_pack_t(const float* x, const float* thr, uint32_t* bits_t, int64_t B,
                               int64_t F, int64_t T, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(x && thr && bits_t && B > 0 && F > 0 && T > 0);
    DL_REQUIRE(Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    dim3 grid((unsigned)dl_ceil_div(Bp, TILE_B), (unsigned)dl_ceil_div(F, TILE_F));
    pack_t_kernel<0><<<grid, PACK_THREADS, 0, dl_cast(stream)>>>(x, thr, 0.f, bits_t, B, F, (int)T,
                                                                Bp / 32);
    return dl_launch_status();
}

DL_EXPORT int64_t dl_swizzled_words(int64_t Bp) { return Bp <= 0 ? 0 : dl_ceil_div(Bp, 1024) * 32; }

DL_EXPORT int dl_bits_swizzle_t(const uint32_t* bits_t, uint32_t* bits_s, int64_t F, int64_t Bp,
                                dl_stream_t stream) {
    DL_REQUIRE(bits_t && bits_s && bits_t != bits_s && F > 0 && Bp > 0 && Bp % DL_BATCH_ALIGN == 0);
    const int64_t G = dl_ceil_div(Bp, 1024);
    const int64_t blocks = dl_min64(dl_ceil_div(F * G, 8), (int64_t)DL_NUM_SMS * 16);
    bits_swizzle_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(bits_t, bits_s, F, Bp / 32, G);
    return dl_launch_status();
}

DL_EXPORT int dl_thermo_pack_s(const float* x, const float* thr, uint32_t* bits_s, int64_t B, int64_t F,
                               int64_t T, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(x && thr && bits_s && B > 0 && F > 0 && T > 0);
    DL_REQUIRE(Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    const int64_t G = dl_ceil_div(Bp, 1024);
    DL_REQUIRE(G <= 0x7fffffff && dl_ceil_div(F, 4) <= 65535);
    // 16-byte loads need whole quads of features per row and aligned rows
    const bool vec4 = F % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
    // small batches: four features per CTA so that the grid still covers the GPU about twice
    const bool narrow = G * dl_ceil_div(F, 8) < 2 * DL_NUM_SMS;
    cudaStream_t s = dl_cast(stream);
    if (narrow) {
        dim3 grid((unsigned)G, (unsigned)dl_ceil_div(F, 4));
        if (vec4) thermo_pack_s_kernel<4, true><<<grid, 128, 0, s>>>(x, thr, bits_s, B, F, (int)T, G);
        else thermo_pack_s_kernel<4, false><<<grid, 128, 0, s>>>(x, thr, bits_s, B, F, (int)T, G);
    } else {
        dim3 grid((unsigned)G, (unsigned)dl_ceil_div(F, 8));
        if (vec4) thermo_pack_s_kernel<8, true><<<grid, 256, 0, s>>>(x, thr, bits_s, B, F, (int)T, G);
        else thermo_pack_s_kernel<8, false><<<grid, 256, 0, s>>>(x, thr, bits_s, B, F, (int)T, G);
    }
    return dl_launch_status();
}

DL_EXPORT int dl_thermo_pack_rows(const float* x, const float* thr, uint32_t* bits, int64_t B,
                                  int64_t F, int64_t T, dl_stream_t stream) {
    DL_REQUIRE(x && thr && bits && B > 0 && F > 0 && T > 0);
    const int64_t Wr = dl_ceil_div(F * T, 32);
    const int blocks = (int)dl_min64(dl_ceil_div(B * Wr * 32, 256), (int64_t)DL_NUM_SMS * 16);
    thermo_pack_rows_kernel<<<blocks, 256, 0, dl_cast(stream)>>>(x, thr, bits, B, F, (int)T, Wr);
    return dl_launch_status();
}

DL_EXPORT int dl_pack_rows_to_t(const float* x, uint32_t* bits_t, int64_t B, int64_t F, int64_t Bp,
                                float threshold, dl_stream_t stream) {
    DL_REQUIRE(x && bits_t && B > 0 && F > 0);
    DL_REQUIRE(Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    dim3 grid((unsigned)dl_ceil_div(Bp, TILE_B), (unsigned)dl_ceil_div(F, TILE_F));
    pack_t_kernel<1><<<grid, PACK_THREADS, 0, dl_cast(stream)>>>(x, nullptr, threshold, bits_t, B, F,
                                                                1, Bp / 32);
    return dl_launch_status();
}

DL_EXPORT int dl_pack_t_to_t(const float* src_t, uint32_t* bits_t, int64_t F, int64_t B, int64_t ld, int64_t Bp,
                             float threshold, dl_stream_t stream) {
    DL_REQUIRE(src_t && bits_t && F > 0 && B > 0 && ld >= B);
    DL_REQUIRE(Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    const int64_t items = F * (Bp / 128);
    if (ld % 4 == 0 && reinterpret_cast<uintptr_t>(src_t) % 16 == 0 && ld >= Bp) {
        const int64_t blocks4 = dl_min64(dl_ceil_div(F * dl_ceil_div(Bp / 128, 4), 8), (int64_t)DL_NUM_SMS * 16);
        pack_t_to_t_vec_kernel<<<(unsigned)blocks4, 256, 0, dl_cast(stream)>>>(src_t, bits_t, F, B, ld, Bp / 32,
                                                                            threshold);
        return dl_launch_status();
    }
    const int64_t blocks = dl_min64(dl_ceil_div(items, 8), (int64_t)DL_NUM_SMS * 16);
    pack_t_to_t_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(src_t, bits_t, F, B, ld, Bp / 32, threshold);
    return dl_launch_status();
}

DL_EXPORT int dl_f32_rows_to_t(const float* rows, float* t, int64_t B, int64_t F, int64_t Bp,
                               dl_stream_t stream) {
    DL_REQUIRE(rows && t && B > 0 && F > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    if (transpose64_ok(rows, t, F, Bp) && dl_ceil_div(F, 64) <= 65535) {
        // source = rows (B x F), destination = t (F x Bp); samples B..Bp-1 are written as zeros
        dim3 grid64((unsigned)(Bp / 64 + (Bp % 64 != 0)), (unsigned)dl_ceil_div(F, 64));
        transpose64_kernel<<<grid64, 256, 0, dl_cast(stream)>>>(rows, t, B, F, F, Bp, F, Bp);
        return dl_launch_status();
    }
    dim3 grid((unsigned)(Bp / 32), (unsigned)dl_ceil_div(F, 32));
    rows_to_t_kernel<<<grid, 256, 0, dl_cast(stream)>>>(rows, t, B, F, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_f32_t_to_rows(const float* t, float* rows, int64_t B, int64_t F, int64_t Bp,
                               dl_stream_t stream) {
    DL_REQUIRE(rows && t && B > 0 && F > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    if (transpose64_ok(rows, t, F, Bp) && dl_ceil_div(B, 64) <= 65535) {
        // source = t (F x Bp), destination = rows (B x F): only the B real samples become rows
        dim3 grid64((unsigned)dl_ceil_div(F, 64), (unsigned)dl_ceil_div(B, 64));
        transpose64_kernel<<<grid64, 256, 0, dl_cast(stream)>>>(t, rows, F, B, Bp, F, Bp, F);
        return dl_launch_status();
    }
    dim3 grid((unsigned)dl_ceil_div(B, 32), (unsigned)dl_ceil_div(F, 32));
    t_to_rows_kernel<<<grid, 256, 0, dl_cast(stream)>>>(t, rows, B, F, Bp);
    return dl_launch_status();
}

DL_EXPORT int dl_bits_t_to_rows(const uint32_t* bits_t, float* rows, int64_t B, int64_t F, int64_t Bp,
                                dl_stream_t stream) {
    DL_REQUIRE(rows && bits_t && B > 0 && F > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    dim3 grid((unsigned)dl_ceil_div(B, 32), (unsigned)dl_ceil_div(F, 32));
    bits_t_to_rows_kernel<<<grid, 256, 0, dl_cast(stream)>>>(bits_t, rows, B, F, Bp / 32);
    return dl_launch_status();
}

DL_EXPORT int dl_bits_rows_to_t(const uint32_t* bits_rows, uint32_t* bits_t, int64_t B, int64_t F,
                                int64_t Wr, int64_t Bp, dl_stream_t stream) {
    DL_REQUIRE(bits_rows && bits_t && B > 0 && F > 0 && Bp >= B && Bp % DL_BATCH_ALIGN == 0);
    DL_REQUIRE(Wr * 32 >= F);
    dim3 grid((unsigned)dl_ceil_div(Bp, 512), (unsigned)dl_ceil_div(dl_ceil_div(F, 32), 8));
    DL_REQUIRE(grid.y <= 65535);
    bits_rows_to_t_kernel<<<grid, 256, 0, dl_cast(stream)>>>(bits_rows, bits_t, B, F, Wr, Bp / 32);
    return dl_launch_status();
}
