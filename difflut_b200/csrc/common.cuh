// Shared helpers for the difflut_b200 kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/difflut_b200.h"

#define DL_EXPORT extern "C" __attribute__((visibility("default")))

// Every entry point validates on the host, launches on the caller's stream and reports
// launch-time errors through cudaPeekAtLastError (no synchronisation, no allocation).
#define DL_REQUIRE(cond)                \
    do {                                \
        if (!(cond)) return DL_ERR_ARG; \
    } while (0)

#define DL_REQUIRE_ALIGNED(p, a)                                              \
    do {                                                                      \
        if ((reinterpret_cast<uintptr_t>(p) % (a)) != 0) return DL_ERR_ALIGN; \
    } while (0)

static inline int dl_launch_status() {
    return cudaPeekAtLastError() == cudaSuccess ? DL_OK : DL_ERR_LAUNCH;
}

static inline cudaStream_t dl_cast(dl_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

static inline int64_t dl_ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int64_t dl_min64(int64_t a, int64_t b) { return a < b ? a : b; }
static inline int64_t dl_max64(int64_t a, int64_t b) { return a > b ? a : b; }

// Number of streaming multiprocessors the grids are sized for (B200: 148).
constexpr int DL_NUM_SMS = 148;

// Spread the 4 low bits of `nib` to the least-significant bit of each byte:
// bit q -> bit 8q.  (1 + 2^7 + 2^14 + 2^21 places every product term on a distinct bit.)
__device__ __forceinline__ uint32_t dl_spread_nibble(uint32_t nib) {
    return (nib * 0x00204081u) & 0x01010101u;
}

// One Adam element update (torch.optim.Adam without weight decay / amsgrad): m <- lerp(m, g, 1-b1),
// v <- v*b2 + (1-b2)*g*g, p <- p - step_size * m / (sqrt(v)/sqrt(bc2) + eps), g = g_raw * gscale.  Every
// operation is written with its rounding spelled out, so that the compiler cannot contract it differently
// in different kernels: the local and the peer-to-peer optimiser kernels produce the same bits.
__device__ __forceinline__ float adam_update(float p, float g_raw, float gscale, float& m, float& v, float step_size,
                                             float bc2_sqrt, float b1, float b2, float eps) {
    const float gi = __fmul_rn(g_raw, gscale);
    m = __fmaf_rn(__fsub_rn(gi, m), __fsub_rn(1.0f, b1), m);
    v = __fmaf_rn(__fmul_rn(__fsub_rn(1.0f, b2), gi), gi, __fmul_rn(v, b2));
    const float denom = __fadd_rn(__fdiv_rn(__fsqrt_rn(v), bc2_sqrt), eps);
    return __fmaf_rn(-step_size, __fdiv_rn(m, denom), p);
}

// Software-pipelined fused DWN backward for n = 6, chunk-interleaved bits and whole 1024-sample blocks
// (dwn_bwd_pipelined.cu); arguments as dl_dwn_bwd_fused_s after validation.  Returns DL_ERR_UNSUPPORTED
// (nothing launched) when a row offset does not fit 32 bits.
int dl_launch_bwd_pipelined(const uint8_t* addr_up, const float* g_up, int64_t gdiv_up, float gscale_up,
                            const float* efd_up, int n_up, const int32_t* inv_ptr, const int32_t* inv_ent,
                            const uint32_t* in_bits, const int32_t* map, float* g_out, uint8_t* addr_out,
                            float* gt, int64_t group_stride, int64_t N, int64_t N_up, int64_t Bp, int64_t Wp,
                            int blocks_per_item, cudaStream_t s);
