// RandomLayer gather on fp32 rows and its scatter-add backward (API-exact `get_mapping`).
//
// Forward is an indexed copy.  The backward replaces the reference's global fp32 atomics
// (difflut/layers/cuda/mapping_cuda_kernel.cu:136-162) by a segmented sum over the inverse map:
// the owner of (b, f) adds the gradient columns listed for feature f in a fixed order.  The forward has a plain
// form (one thread per element) and a shared-memory staged form that the entry point prefers when a row fits;
// both are exact copies.  The backward has two forms as well.  dl_gather_rows_bwd takes the inverse map as CSR
// and gives one thread a feature and four rows; it fetches a 32-byte sector for every 4-byte gradient AND for
// every 4-byte entry (neighbouring features' lists lie 60 bytes apart), and staging the gradient row in shared
// memory alone did not help it (0.59 - 0.92 ms against 0.71 ms at the first layer's width, 2048 rows).
// dl_gather_rows_bwd_ell takes the entries interleaved by feature and stages the gradient: both streams coalesced.
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

// Column-tiled backward over an entry table interleaved by feature: ell[j * F + f] = the j-th column that
// feature f collects (ascending), -1 when f has fewer.  A CTA takes one gradient row at a time and walks it in
// tiles of TB_COLS columns: the tile is copied into shared memory in coalesced 16-byte pieces; a thread owns
// TB_FEATS features (f = tid + k * TB_THREADS, so the lanes of a warp read neighbouring table entries) and, in
// rounds over all of them, consumes the pending entry of every feature whose column lies in the tile and
// requests that feature's next entry.  Every gradient and every entry is read once per pass, coalesced; a
// feature's gradients are added in ascending column order, as in the plain kernel: same bits.
constexpr int TB_THREADS = 512, TB_FEATS = 13, TB_COLS = 10240;

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}

// The tile of the step after the current one is copied global -> shared asynchronously (cp.async, two tile
// buffers) while the current tile is consumed, across row boundaries too, so a CTA's loads and look-ups overlap.
__global__ void __launch_bounds__(TB_THREADS, 2)
gather_rows_bwd_ell_kernel(const float* __restrict__ g, const int32_t* __restrict__ ell, int max_deg,
                           float* __restrict__ gx, int64_t B, int64_t F, int64_t M, int64_t f_base) {
    extern __shared__ float tile_s[];  // [2][TB_COLS] gradient tiles, then [TB_FEATS][TB_THREADS] running sums
    const int tid = threadIdx.x;
    float* acc_s = tile_s + 2 * TB_COLS + tid;  // acc_s[k * TB_THREADS]: private to the thread (registers are short)
    // entries are addressed as ellf[off]: off = j * F + k * TB_THREADS in 32 bits (the launcher checks the range)
    const int32_t* ellf = ell + f_base + tid;
    const uint32_t F32 = (uint32_t)F, limit = (uint32_t)max_deg * (uint32_t)F;
    const int tiles = (int)((M + TB_COLS - 1) / TB_COLS);

    auto issue = [&](int buf, int64_t b, int t) {  // request tile t of row b into buffer buf (one commit group)
        if (b < B) {
            const int64_t c0 = (int64_t)t * TB_COLS;
            const int64_t c1 = c0 + TB_COLS < M ? c0 + TB_COLS : M;
            const float* src = g + b * M + c0;   // M % 4 == 0 and c0 % 4 == 0: 16-byte aligned
            float* dst = tile_s + buf * TB_COLS;
            const int quads = (int)((c1 - c0) >> 2);
            for (int q = tid; q < quads; q += TB_THREADS) cp_async16(dst + 4 * q, src + 4 * q);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    int64_t b = blockIdx.x;
    int t = 0, buf = 0;
    issue(0, b, 0);
    uint32_t off[TB_FEATS];  // offset of the feature's pending entry
    int c[TB_FEATS];         // its column, -1 = the feature has no more entries
    while (b < B) {
        // the step after this one
        int64_t nb = b;
        int nt = t + 1;
        if (nt == tiles) { nt = 0; nb = b + gridDim.x; }
        issue(buf ^ 1, nb, nt);
        if (t == 0) {
#pragma unroll
            for (int k = 0; k < TB_FEATS; ++k) {
                acc_s[k * TB_THREADS] = 0.f;
                off[k] = (uint32_t)k * TB_THREADS;
                c[k] = (f_base + tid + (int64_t)k * TB_THREADS < F && max_deg > 0) ? __ldg(ellf + off[k]) : -1;
            }
        }
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group has landed
        __syncthreads();
        const float* tile = tile_s + buf * TB_COLS;
        const int lo = t * TB_COLS;
        const int hi = lo + TB_COLS < (int)M ? lo + TB_COLS : (int)M;
        bool more = true;
        while (more) {
            more = false;
#pragma unroll
            for (int k = 0; k < TB_FEATS; ++k) {
                if (c[k] >= 0 && c[k] < hi) {
                    acc_s[k * TB_THREADS] += tile[c[k] - lo];
                    off[k] += F32;
                    c[k] = off[k] < limit ? __ldg(ellf + off[k]) : -1;
                    more = true;
                }
            }
        }
        if (nt == 0) {  // the row is complete
#pragma unroll
            for (int k = 0; k < TB_FEATS; ++k) {
                const int64_t f = f_base + tid + (int64_t)k * TB_THREADS;
                if (f < F) gx[b * F + f] = acc_s[k * TB_THREADS];
            }
        }
        __syncthreads();  // this buffer is requested again two steps from now
        b = nb;
        t = nt;
        buf ^= 1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

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

DL_EXPORT int dl_gather_rows_bwd_ell(const float* g, const int32_t* ell, int64_t max_deg, float* gx, int64_t B,
                                     int64_t F, int64_t N, int64_t n, dl_stream_t stream) {
    DL_REQUIRE(g && ell && gx && B > 0 && F > 0 && N > 0 && n > 0 && max_deg >= 0 && max_deg < ((int64_t)1 << 20));
    const int64_t M = N * n;
    DL_REQUIRE(M % 4 == 0 && M < ((int64_t)1 << 31) && (max_deg + 1) * F < ((int64_t)1 << 31));
    DL_REQUIRE_ALIGNED(g, 16);
    const size_t smem = (2 * (size_t)TB_COLS + (size_t)TB_FEATS * TB_THREADS) * sizeof(float);
    if (cudaFuncSetAttribute(gather_rows_bwd_ell_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
        return DL_ERR_LAUNCH;
    const int64_t per_pass = (int64_t)TB_THREADS * TB_FEATS;
    const int64_t blocks = dl_min64(B, (int64_t)DL_NUM_SMS * 2);
    for (int64_t f_base = 0; f_base < F; f_base += per_pass)
        gather_rows_bwd_ell_kernel<<<(unsigned)blocks, TB_THREADS, smem, dl_cast(stream)>>>(g, ell, (int)max_deg, gx, B,
                                                                                          F, M, f_base);
    return dl_launch_status();
}
