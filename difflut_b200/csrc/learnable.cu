// LearnableLayer soft connectivity: row softmax + a tcgen05 / TMA tensor-core GEMM.
//
// The reference computes `x @ softmax(W/tau, -1).T` with F.softmax + torch.matmul
// (difflut/layers/learnable_layer.py:253-255) and lets autograd produce the two backward GEMMs.
// Here the three contractions run on one kernel, C[M,N] (fp32) = A[M,K] * B[N,K]^T with bf16
// operands: TMA (cp.async.bulk.tensor) stages 128x64 / 256x64 operand tiles in 128-byte-swizzled
// shared memory, one elected thread issues tcgen05.mma (kind::f16, fp32 accumulator in tensor
// memory), and four epilogue warps read the accumulator back with tcgen05.ld.  CTAs are persistent
// and the accumulator is double-buffered, so the epilogue of a tile overlaps the next tile's MMAs.
// No cluster, no multicast.  Every wait on an mbarrier is bounded: when a wait runs out the kernel
// records where it gave up in `status` and leaves (after freeing its tensor memory).
#include <cuda.h>
#include <cuda_bf16.h>

#include <atomic>

#include "common.cuh"

namespace {

constexpr int BM = 128;          // accumulator rows = TMEM lanes
constexpr int BN = 256;          // accumulator columns = TMEM columns
constexpr int BK = 64;           // 64 bf16 = 128 bytes: one swizzle row
constexpr int UMMA_K = 16;       // K per tcgen05.mma for 16-bit operands
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;      // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // every wait gives up after about one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait on a phase parity; false when the limit ran out or another role of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    const uint32_t addr = smem_u32(bar);
    const long long start = clock64();
    for (uint32_t it = 0;; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((it & 63u) == 63u && (*abort_flag != 0 || clock64() - start > WAIT_LIMIT_CYCLES)) return false;
    }
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes, 128-byte swizzle:
// start address >> 4, stride between 8-row groups = 1024 bytes, descriptor version 1, layout 2.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                   // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;        // stride byte offset
    d |= (uint64_t)1 << 46;                   // descriptor version
    d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D = f32, A = B = bf16, both K-major, N and M of the tile.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// Persistent kernel: each CTA (one per SM) walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The
// accumulator is double-buffered in tensor memory (2 x 256 columns), so the epilogue warps drain
// tile t while the MMA thread already accumulates tile t+1; the TMA / MMA stage ring runs across
// tile boundaries without draining.
// status[0] = 0 ok, otherwise (role << 8 | stage) of the wait that gave up.
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    float* __restrict__ C, uint32_t* __restrict__ Cbits, int64_t Wp, float threshold, int M, int N,
                    int K, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;    // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;     // [2] epilogue -> MMA (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the operand with fewer row tiles is the fast tile index, so CTAs that run together share the
    // tiles of the large operand's current row block and the small operand is re-read from L2
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n;
    const bool m_fast = tiles_m <= tiles_n;
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // all 512 columns of tensor memory: two 128 x 256 fp32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)(2 * BN))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t kc = 0;  // k-blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < total_tiles && *abort_flag == 0; tile += gridDim.x) {
                const int tile_m = m_fast ? tile % tiles_m : tile / tiles_n;
                const int tile_n = m_fast ? tile / tiles_m : tile % tiles_n;
                for (int kb = 0; kb < kblocks; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    const uint32_t use = kc / STAGES;
                    if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1, abort_flag)) {
                        atomicCAS(status, 0, (1 << 8) | s);
                        *abort_flag = 1;
                        break;
                    }
                    uint8_t* a_dst = tiles + s * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, &full[s], kb * BK, tile_m * BM);
                    tma_load_2d(b_dst, &map_b, &full[s], kb * BK, tile_n * BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(BM, BN);
            uint32_t kc = 0, it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && *abort_flag == 0; tile += gridDim.x, ++it) {
                const uint32_t buf = it & 1, useb = it >> 1;
                if (useb > 0 && !mbar_wait(&acc_empty[buf], (useb - 1) & 1, abort_flag)) {
                    atomicCAS(status, 0, (4 << 8) | buf);
                    *abort_flag = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    const uint32_t use = kc / STAGES;
                    if (!mbar_wait(&full[s], use & 1, abort_flag)) {
                        atomicCAS(status, 0, (2 << 8) | s);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // inside the 128-byte swizzle row the next 16 elements start 32 bytes further
                        const uint64_t adesc = umma_desc_k_major_sw128(a_addr + k * UMMA_K * 2);
                        const uint64_t bdesc = umma_desc_k_major_sw128(b_addr + k * UMMA_K * 2);
                        umma_bf16(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);  // the stage is free again once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[buf]);  // arrives when every MMA of this tile has finished
            }
        }
    } else {
        // epilogue: warp w may read TMEM lanes 32*(w%4) .. +31; one accumulator row per thread
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int tile_m = m_fast ? tile % tiles_m : tile / tiles_n;
            const int tile_n = m_fast ? tile / tiles_m : tile % tiles_n;
            const uint32_t buf = it & 1, useb = it >> 1;
            const int64_t grow = (int64_t)tile_m * BM + row;
            if (!mbar_wait(&acc_full[buf], useb & 1, abort_flag)) {
                if (lane == 0) {
                    atomicCAS(status, 0, (3 << 8) | buf);
                    *abort_flag = 1;
                }
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                      "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                      "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                      "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (grow < M && Cbits != nullptr) {
                    // packed result: the thread holds 32 consecutive columns of its row = one word of that row
                    const int64_t gcol = (int64_t)tile_n * BN + c0;
                    if (gcol < N) {
                        uint32_t word = 0;
#pragma unroll
                        for (int q = 0; q < 32; ++q)
                            word |= (gcol + q < N && __uint_as_float(r[q]) >= threshold) ? (1u << q) : 0u;
                        Cbits[grow * Wp + (gcol >> 5)] = word;
                    }
                } else if (grow < M) {
                    const int64_t gcol = (int64_t)tile_n * BN + c0;
                    float* dst = C + grow * N + gcol;
                    if (gcol + 32 <= N && (N & 3) == 0) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            reinterpret_cast<float4*>(dst)[q] =
                                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                            __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                    } else {
#pragma unroll
                        for (int q = 0; q < 32; ++q)
                            if (gcol + q < N) dst[q] = __uint_as_float(r[q]);
                    }
                }
            }
            // this warp has read its quarter of the buffer: hand it back to the MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN))
                     : "memory");
    }
}

// bf16 [rows][cols] row-major tensor map with a (box_rows x 64) box and 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    // the driver entry point is looked up through the runtime, so the library itself does not link
    // against libcuda and still loads on a machine without a driver
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::atomic<encode_fn> cached{nullptr};  // looked up once; concurrent first calls resolve the same pointer
    encode_fn encode = cached.load(std::memory_order_acquire);
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            fn == nullptr)
            return DL_ERR_LAUNCH;
        encode = reinterpret_cast<encode_fn>(fn);
        cached.store(encode, std::memory_order_release);
    }
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? DL_OK : DL_ERR_ARG;
}

// ------------------------------------------------------------------------------------------
// softmax rows, conversions
// ------------------------------------------------------------------------------------------

__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, u) : v + u;
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nw = blockDim.x >> 5;
    float r = is_max ? -INFINITY : 0.f;
    for (int w = 0; w < nw; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
    return r;
}

// one CTA per row: S = softmax(W / tau) - center written as bf16 hi (+ optional lo = bf16(S - hi))
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const float* __restrict__ W, float inv_tau, float center, __nv_bfloat16* __restrict__ S_hi,
                    __nv_bfloat16* __restrict__ S_lo, int64_t ld_out, int64_t I) {
    __shared__ float scratch[8];
    const int64_t row = blockIdx.x;
    const float* w = W + row * I;
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < I; i += blockDim.x) mx = fmaxf(mx, w[i] * inv_tau);
    mx = block_reduce(mx, scratch, true);
    float sum = 0.f;
    for (int64_t i = threadIdx.x; i < I; i += blockDim.x) sum += expf(w[i] * inv_tau - mx);
    sum = block_reduce(sum, scratch, false);
    const float inv = 1.0f / sum;
    for (int64_t i = threadIdx.x; i < I; i += blockDim.x) {
        const float s = expf(w[i] * inv_tau - mx) * inv - center;
        const __nv_bfloat16 hi = __float2bfloat16(s);
        S_hi[row * ld_out + i] = hi;
        if (S_lo != nullptr) S_lo[row * ld_out + i] = __float2bfloat16(s - __bfloat162float(hi));
    }
}

// gW[row] = S * (gS - sum(gS * S)) / tau with S recomputed from W in fp32
__global__ void __launch_bounds__(256)
softmax_bwd_rows_kernel(const float* __restrict__ W, const float* __restrict__ gS, float inv_tau,
                        float* __restrict__ gW, int64_t I) {
    __shared__ float scratch[8];
    const int64_t row = blockIdx.x;
    const float* w = W + row * I;
    const float* g = gS + row * I;
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < I; i += blockDim.x) mx = fmaxf(mx, w[i] * inv_tau);
    mx = block_reduce(mx, scratch, true);
    float sum = 0.f, dot = 0.f;
    for (int64_t i = threadIdx.x; i < I; i += blockDim.x) {
        const float e = expf(w[i] * inv_tau - mx);
        sum += e;
        dot += e * g[i];
    }
    sum = block_reduce(sum, scratch, false);
    dot = block_reduce(dot, scratch, false);
    const float inv = 1.0f / sum;
    const float mean = dot * inv;
    for (int64_t i = threadIdx.x; i < I; i += blockDim.x) {
        const float s = expf(w[i] * inv_tau - mx) * inv;
        gW[row * I + i] = s * (g[i] - mean) * inv_tau;
    }
}

// Register-resident variants for rows of up to 256 * 4 * SM_MAXQ elements (a multiple of 4): the row is read
// once with 16-byte loads, every exponential is evaluated once, outputs leave as 8- / 16-byte stores.
constexpr int SM_MAXQ = 8;

__device__ __forceinline__ uint2 pack_bf16x4(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 out;
    out.x = *reinterpret_cast<uint32_t*>(&lo);
    out.y = *reinterpret_cast<uint32_t*>(&hi);
    return out;
}

// QN: 16-byte pieces per thread (the row has at most 256 * QN of them); the launcher picks the smallest that fits,
// so a 4096-wide row holds 16 values per thread instead of 32 and more rows are resident per SM.
template <int QN>
__global__ void __launch_bounds__(256)
softmax_rows_vec_kernel(const float* __restrict__ W, float inv_tau, float center, __nv_bfloat16* __restrict__ S_hi,
                        __nv_bfloat16* __restrict__ S_lo, int64_t ld_out, int I4) {
    __shared__ float scratch[8];
    const int64_t row = blockIdx.x;
    const float4* w = reinterpret_cast<const float4*>(W + row * (int64_t)I4 * 4);
    float4 v[QN];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < QN; ++k) {
        const int q = threadIdx.x + k * 256;
        if (q < I4) {
            const float4 t = __ldg(w + q);
            v[k] = make_float4(t.x * inv_tau, t.y * inv_tau, t.z * inv_tau, t.w * inv_tau);
            mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
        } else {
            v[k] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
    }
    mx = block_reduce(mx, scratch, true);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < QN; ++k) {
        v[k].x = expf(v[k].x - mx); v[k].y = expf(v[k].y - mx);
        v[k].z = expf(v[k].z - mx); v[k].w = expf(v[k].w - mx);
        sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    sum = block_reduce(sum, scratch, false);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int k = 0; k < QN; ++k) {
        const int q = threadIdx.x + k * 256;
        if (q < I4) {
            const float a = v[k].x * inv - center, b = v[k].y * inv - center, c = v[k].z * inv - center,
                        d = v[k].w * inv - center;
            const uint2 hi = pack_bf16x4(a, b, c, d);
            *reinterpret_cast<uint2*>(S_hi + row * ld_out + 4 * q) = hi;
            if (S_lo != nullptr) {
                const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&hi.x);
                const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&hi.y);
                *reinterpret_cast<uint2*>(S_lo + row * ld_out + 4 * q) =
                    pack_bf16x4(a - __low2float(h0), b - __high2float(h0), c - __low2float(h1), d - __high2float(h1));
            }
        }
    }
}

template <int QN>
__global__ void __launch_bounds__(256)
softmax_bwd_rows_vec_kernel(const float* __restrict__ W, const float* __restrict__ gS, float inv_tau,
                            float* __restrict__ gW, int I4) {
    __shared__ float scratch[8];
    const int64_t row = blockIdx.x;
    const float4* w = reinterpret_cast<const float4*>(W + row * (int64_t)I4 * 4);
    const float4* g = reinterpret_cast<const float4*>(gS + row * (int64_t)I4 * 4);
    float4 v[QN], gg[QN];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < QN; ++k) {
        const int q = threadIdx.x + k * 256;
        if (q < I4) {
            const float4 t = __ldg(w + q);
            gg[k] = __ldg(g + q);
            v[k] = make_float4(t.x * inv_tau, t.y * inv_tau, t.z * inv_tau, t.w * inv_tau);
            mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
        } else {
            v[k] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            gg[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    mx = block_reduce(mx, scratch, true);
    float sum = 0.f, dot = 0.f;
#pragma unroll
    for (int k = 0; k < QN; ++k) {
        v[k].x = expf(v[k].x - mx); v[k].y = expf(v[k].y - mx);
        v[k].z = expf(v[k].z - mx); v[k].w = expf(v[k].w - mx);
        sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        dot += (v[k].x * gg[k].x + v[k].y * gg[k].y) + (v[k].z * gg[k].z + v[k].w * gg[k].w);
    }
    sum = block_reduce(sum, scratch, false);
    dot = block_reduce(dot, scratch, false);
    const float inv = 1.0f / sum;
    const float mean = dot * inv;
    float4* out = reinterpret_cast<float4*>(gW + row * (int64_t)I4 * 4);
#pragma unroll
    for (int k = 0; k < QN; ++k) {
        const int q = threadIdx.x + k * 256;
        if (q < I4) {
            float4 r;
            r.x = v[k].x * inv * (gg[k].x - mean) * inv_tau;
            r.y = v[k].y * inv * (gg[k].y - mean) * inv_tau;
            r.z = v[k].z * inv * (gg[k].z - mean) * inv_tau;
            r.w = v[k].w * inv * (gg[k].w - mean) * inv_tau;
            out[q] = r;
        }
    }
}

// fp32 (rows, cols) -> bf16, written at dst[r * ld + c] (or transposed: dst[c * ld + r]); optional
// residual lo = bf16(x - hi) written at the same place of dst_lo
__global__ void __launch_bounds__(256)
to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, __nv_bfloat16* __restrict__ dst_lo,
               int64_t rows, int64_t cols, int64_t ld, bool transpose) {
    __shared__ float tile[32][33];
    const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int64_t rr = r0 + r, cc = c0 + tx;
        tile[r][tx] = (rr < rows && cc < cols) ? src[rr * cols + cc] : 0.f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        float v;
        int64_t off;
        bool ok;
        if (!transpose) {
            const int64_t rr = r0 + r, cc = c0 + tx;
            v = tile[r][tx]; off = rr * ld + cc; ok = rr < rows && cc < cols;
        } else {
            const int64_t cc = c0 + r, rr = r0 + tx;
            v = tile[tx][r]; off = cc * ld + rr; ok = rr < rows && cc < cols;
        }
        if (ok) {
            const __nv_bfloat16 hi = __float2bfloat16(v);
            dst[off] = hi;
            if (dst_lo != nullptr) dst_lo[off] = __float2bfloat16(v - __bfloat162float(hi));
        }
    }
}

// The common case without transposition or residual: four elements per thread, 16-byte loads, 8-byte stores.
__global__ void __launch_bounds__(256)
to_bf16_vec_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t rows, int64_t cq,
                   int64_t ld) {
    const int64_t total = rows * cq;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / cq, q = t - r * cq;
        const float4 v = __ldg(reinterpret_cast<const float4*>(src) + t);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 out;
        out.x = *reinterpret_cast<uint32_t*>(&a);
        out.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(dst + r * ld + q * 4) = out;
    }
}

// bf16 (rows, cols) with row pitch ld_src -> transposed bf16 (cols, rows) with row pitch ld_dst
__global__ void __launch_bounds__(256)
bf16_transpose_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t rows,
                      int64_t cols, int64_t ld_src, int64_t ld_dst) {
    __shared__ __nv_bfloat16 tile[64][66];
    const int64_t c0 = (int64_t)blockIdx.x * 64, r0 = (int64_t)blockIdx.y * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (int r = ty; r < 64; r += 4) {
        const int64_t rr = r0 + r, cc = c0 + tx;
        tile[r][tx] = (rr < rows && cc < cols) ? src[rr * ld_src + cc] : __float2bfloat16(0.f);
    }
    __syncthreads();
    for (int c = ty; c < 64; c += 4) {
        const int64_t cc = c0 + c, rr = r0 + tx;
        if (cc < cols && rr < rows) dst[cc * ld_dst + rr] = tile[tx][c];
    }
}

}  // namespace

DL_EXPORT int dl_gemm_bf16_tn(const void* A, const void* B, float* C, int64_t M, int64_t N, int64_t K,
                              int* status, dl_stream_t stream) {
    DL_REQUIRE(A && B && C && status && M > 0 && N > 0 && K > 0);
    DL_REQUIRE(M < ((int64_t)1 << 31) && N < ((int64_t)1 << 31) && K < ((int64_t)1 << 31));
    DL_REQUIRE_ALIGNED(A, 16);
    DL_REQUIRE_ALIGNED(B, 16);
    DL_REQUIRE_ALIGNED(C, 16);
    if (K % 8 != 0) return DL_ERR_ALIGN;  // tensor-map row pitch must be a multiple of 16 bytes
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, A, M, K, BM);
    if (rc != DL_OK) return rc;
    rc = make_map(&map_b, B, N, K, BN);
    if (rc != DL_OK) return rc;
    cudaFuncSetAttribute(gemm_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    const int64_t gx = dl_ceil_div(N, BN), gy = dl_ceil_div(M, BM);
    DL_REQUIRE(gx * gy < ((int64_t)1 << 31));
    dim3 grid((unsigned)dl_min64(gx * gy, DL_NUM_SMS));
    gemm_bf16_tn_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, dl_cast(stream)>>>(map_a, map_b, C, nullptr, 0, 0.f, (int)M,
                                                                           (int)N, (int)K, status);
    return dl_launch_status();
}

DL_EXPORT int dl_gemm_bf16_tn_bits(const void* A, const void* B, uint32_t* bits, int64_t M, int64_t N, int64_t K,
                                   int64_t Wp, float threshold, int* status, dl_stream_t stream) {
    DL_REQUIRE(A && B && bits && status && M > 0 && N > 0 && K > 0 && Wp * 32 >= N);
    DL_REQUIRE(M < ((int64_t)1 << 31) && N < ((int64_t)1 << 31) && K < ((int64_t)1 << 31));
    DL_REQUIRE_ALIGNED(A, 16);
    DL_REQUIRE_ALIGNED(B, 16);
    if (K % 8 != 0) return DL_ERR_ALIGN;  // tensor-map row pitch must be a multiple of 16 bytes
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, A, M, K, BM);
    if (rc != DL_OK) return rc;
    rc = make_map(&map_b, B, N, K, BN);
    if (rc != DL_OK) return rc;
    cudaFuncSetAttribute(gemm_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    const int64_t gx = dl_ceil_div(N, BN), gy = dl_ceil_div(M, BM);
    DL_REQUIRE(gx * gy < ((int64_t)1 << 31));
    dim3 grid((unsigned)dl_min64(gx * gy, DL_NUM_SMS));
    gemm_bf16_tn_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, dl_cast(stream)>>>(map_a, map_b, nullptr, bits, Wp, threshold,
                                                                           (int)M, (int)N, (int)K, status);
    return dl_launch_status();
}

static int softmax_rows_launch(const float* W, float tau, float center, void* S_hi, void* S_lo, int64_t ld_out,
                               int64_t M, int64_t I, dl_stream_t stream) {
    const bool aligned = reinterpret_cast<uintptr_t>(W) % 16 == 0 && reinterpret_cast<uintptr_t>(S_hi) % 8 == 0 &&
                         (S_lo == nullptr || reinterpret_cast<uintptr_t>(S_lo) % 8 == 0);
    if (aligned && I % 4 == 0 && ld_out % 4 == 0 && I <= 256 * 4 * SM_MAXQ) {
        __nv_bfloat16* hi = static_cast<__nv_bfloat16*>(S_hi);
        __nv_bfloat16* lo = static_cast<__nv_bfloat16*>(S_lo);
        const int I4 = (int)(I / 4);
        const unsigned rows = (unsigned)M;
        cudaStream_t st = dl_cast(stream);
        if (I4 <= 256) softmax_rows_vec_kernel<1><<<rows, 256, 0, st>>>(W, 1.0f / tau, center, hi, lo, ld_out, I4);
        else if (I4 <= 512) softmax_rows_vec_kernel<2><<<rows, 256, 0, st>>>(W, 1.0f / tau, center, hi, lo, ld_out, I4);
        else if (I4 <= 1024) softmax_rows_vec_kernel<4><<<rows, 256, 0, st>>>(W, 1.0f / tau, center, hi, lo, ld_out, I4);
        else softmax_rows_vec_kernel<SM_MAXQ><<<rows, 256, 0, st>>>(W, 1.0f / tau, center, hi, lo, ld_out, I4);
        return dl_launch_status();
    }
    softmax_rows_kernel<<<(unsigned)M, 256, 0, dl_cast(stream)>>>(W, 1.0f / tau, center,
                                                                 static_cast<__nv_bfloat16*>(S_hi),
                                                                 static_cast<__nv_bfloat16*>(S_lo), ld_out, I);
    return dl_launch_status();
}

DL_EXPORT int dl_softmax_rows_bf16(const float* W, float tau, void* S_hi, void* S_lo, int64_t ld_out, int64_t M,
                                   int64_t I, dl_stream_t stream) {
    DL_REQUIRE(W && S_hi && M > 0 && I > 0 && tau > 0.f && ld_out >= I);
    return softmax_rows_launch(W, tau, 0.f, S_hi, S_lo, ld_out, M, I, stream);
}

// Centred single-pass operands.  A softmax row sums to one, so S = 1/I + D with small D when the selection is
// close to uniform, which is when the contraction's result sits near the 0.5 threshold of the nodes that read it:
//   x . S^T = (sum_i x_i) / I + x . D^T.
// D is what bf16 rounds (its error is relative to D, not to S), and the first term enters the same GEMM
// through three extra K columns: the row of D carries 1, 1, 1 there and the row of x its own sum / I as a
// three-piece bf16 split (24 bits).  The two entry points below write those columns.
__global__ void fill_ones_cols_kernel(__nv_bfloat16* __restrict__ S, int64_t ld, int64_t M, int64_t col0, int ones,
                                      int ext) {
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < M * ext;
         t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = t / ext;
        const int c = (int)(t - row * ext);
        S[row * ld + col0 + c] = __float2bfloat16(c < ones ? 1.0f : 0.0f);
    }
}

// one warp per row: fixed-order sum of the row's bf16 values, times `scale`, split into three bf16 pieces
__global__ void __launch_bounds__(256)
row_sum_split_kernel(__nv_bfloat16* __restrict__ A, int64_t ld, int64_t rows, int64_t cols, int64_t col0, float scale,
                     int ext) {
    const int lane = threadIdx.x & 31;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    const __nv_bfloat16* a = A + row * ld;
    float acc = 0.f;
    for (int64_t i = lane; i < cols; i += 32) acc += __bfloat162float(a[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    const float t = acc * scale;
    const __nv_bfloat16 p0 = __float2bfloat16(t);
    const float r1 = t - __bfloat162float(p0);
    const __nv_bfloat16 p1 = __float2bfloat16(r1);
    const __nv_bfloat16 p2 = __float2bfloat16(r1 - __bfloat162float(p1));
    for (int c = lane; c < ext; c += 32) {
        __nv_bfloat16 v = __float2bfloat16(0.f);
        if (c == 0) v = p0;
        else if (c == 1) v = p1;
        else if (c == 2) v = p2;
        A[row * ld + col0 + c] = v;
    }
}

DL_EXPORT int dl_softmax_rows_centered_bf16(const float* W, float tau, void* S_c, int64_t ld_out, int64_t M, int64_t I,
                                            int64_t ext_col, int64_t ext, dl_stream_t stream) {
    DL_REQUIRE(W && S_c && M > 0 && I > 0 && tau > 0.f && ext >= 3 && ext <= 1024 && ext_col >= I &&
               ld_out >= ext_col + ext);
    const int rc = softmax_rows_launch(W, tau, 1.0f / (float)I, S_c, nullptr, ld_out, M, I, stream);
    if (rc != DL_OK) return rc;
    const int64_t blocks = dl_min64(dl_ceil_div(M * ext, 256), (int64_t)DL_NUM_SMS * 8);
    fill_ones_cols_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(static_cast<__nv_bfloat16*>(S_c), ld_out, M,
                                                                       ext_col, 3, (int)ext);
    return dl_launch_status();
}

DL_EXPORT int dl_row_sum_split_bf16(void* A, int64_t ld, int64_t rows, int64_t cols, int64_t ext_col, float scale,
                                    int64_t ext, dl_stream_t stream) {
    DL_REQUIRE(A && rows > 0 && cols > 0 && ext >= 3 && ext <= 1024 && ext_col >= cols && ld >= ext_col + ext);
    const int64_t blocks = dl_ceil_div(rows * 32, 256);
    DL_REQUIRE(blocks < ((int64_t)1 << 31));
    row_sum_split_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(static_cast<__nv_bfloat16*>(A), ld, rows, cols,
                                                                      ext_col, scale, (int)ext);
    return dl_launch_status();
}

DL_EXPORT int dl_softmax_bwd_rows(const float* W, const float* gS, float tau, float* gW, int64_t M, int64_t I,
                                  dl_stream_t stream) {
    DL_REQUIRE(W && gS && gW && M > 0 && I > 0 && tau > 0.f);
    if (I % 4 == 0 && I <= 256 * 4 * SM_MAXQ && reinterpret_cast<uintptr_t>(W) % 16 == 0 &&
        reinterpret_cast<uintptr_t>(gS) % 16 == 0 && reinterpret_cast<uintptr_t>(gW) % 16 == 0) {
        const int I4 = (int)(I / 4);
        const unsigned rows = (unsigned)M;
        cudaStream_t st = dl_cast(stream);
        if (I4 <= 256) softmax_bwd_rows_vec_kernel<1><<<rows, 256, 0, st>>>(W, gS, 1.0f / tau, gW, I4);
        else if (I4 <= 512) softmax_bwd_rows_vec_kernel<2><<<rows, 256, 0, st>>>(W, gS, 1.0f / tau, gW, I4);
        else if (I4 <= 1024) softmax_bwd_rows_vec_kernel<4><<<rows, 256, 0, st>>>(W, gS, 1.0f / tau, gW, I4);
        else softmax_bwd_rows_vec_kernel<SM_MAXQ><<<rows, 256, 0, st>>>(W, gS, 1.0f / tau, gW, I4);
        return dl_launch_status();
    }
    softmax_bwd_rows_kernel<<<(unsigned)M, 256, 0, dl_cast(stream)>>>(W, gS, 1.0f / tau, gW, I);
    return dl_launch_status();
}

DL_EXPORT int dl_f32_to_bf16(const float* src, void* dst_hi, void* dst_lo, int64_t rows, int64_t cols, int64_t ld,
                             int transpose, dl_stream_t stream) {
    DL_REQUIRE(src && dst_hi && rows > 0 && cols > 0 && ld >= (transpose ? rows : cols));
    if (!transpose && dst_lo == nullptr && cols % 4 == 0 && ld % 4 == 0 &&
        reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst_hi) % 8 == 0) {
        const int64_t blocks = dl_min64(dl_ceil_div(rows * (cols / 4), 256), (int64_t)DL_NUM_SMS * 16);
        to_bf16_vec_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(src, static_cast<__nv_bfloat16*>(dst_hi),
                                                                        rows, cols / 4, ld);
        return dl_launch_status();
    }
    dim3 grid((unsigned)dl_ceil_div(cols, 32), (unsigned)dl_ceil_div(rows, 32));
    DL_REQUIRE(grid.y <= 65535);
    to_bf16_kernel<<<grid, 256, 0, dl_cast(stream)>>>(src, static_cast<__nv_bfloat16*>(dst_hi),
                                                     static_cast<__nv_bfloat16*>(dst_lo), rows, cols, ld, transpose != 0);
    return dl_launch_status();
}

DL_EXPORT int dl_bf16_transpose(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src,
                                int64_t ld_dst, dl_stream_t stream) {
    DL_REQUIRE(src && dst && rows > 0 && cols > 0 && ld_src >= cols && ld_dst >= rows);
    dim3 grid((unsigned)dl_ceil_div(cols, 64), (unsigned)dl_ceil_div(rows, 64));
    DL_REQUIRE(grid.y <= 65535);
    bf16_transpose_kernel<<<grid, 256, 0, dl_cast(stream)>>>(static_cast<const __nv_bfloat16*>(src),
                                                            static_cast<__nv_bfloat16*>(dst), rows, cols, ld_src, ld_dst);
    return dl_launch_status();
}
