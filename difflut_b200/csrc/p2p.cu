// Data-parallel optimiser step over NVLink peer memory: gradient all-reduce, Adam and parameter
// broadcast in one kernel.
//
// Every rank (one process per GPU) maps the other ranks' gradient and parameter buffers (CUDA IPC, plain
// peer pointers: no multicast object is created or used).  Rank r owns slice r of the flat parameter
// vector: it sums that slice of all ranks' gradients with peer loads (fixed rank order), applies Adam
// with its own slice of the moments, and stores the new parameters into every rank's parameter buffer.
// Each element is therefore reduced and updated exactly once and all ranks end up with identical bits;
// the moments exist only on the owner.  Compared with an all-reduce followed by a full Adam on every rank
// this moves the same bytes over NVLink but does 1/world of the optimiser work and has no library launch
// in the step.
//
// Two barriers bracket the kernel: before it (every rank's gradients are complete) and after it (every
// rank's parameter stores have landed before anyone's next forward).  A barrier is a tiny kernel: thread p
// publishes this rank's epoch into rank p's flag array (system-scope release) and waits until rank p's
// epoch shows up in its own array.  Every wait is bounded by a wall-clock limit; on expiry the kernel
// records it in a status word and returns, so a missing peer can never hang the GPU.
#include <cstdlib>

#include "common.cuh"

namespace {

struct PeerTable {
    void* ptr[DL_MAX_PEERS];
};

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void store_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int load_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// flags of rank q: int[DL_MAX_PEERS]; slot p is written by rank p only.  ctrl (local): [0] = epoch,
// [1] = status (0 = fine, else 1 + the first peer that did not arrive in time).
__global__ void p2p_barrier_kernel(PeerTable flags, int rank, int world, int* __restrict__ ctrl,
                                   uint64_t timeout_ns) {
    __shared__ int epoch;
    if (threadIdx.x == 0) epoch = ctrl[0] + 1;
    __syncthreads();
    const int e = epoch;
    const int p = threadIdx.x;
    if (p < world) {
        __threadfence_system();  // everything earlier kernels of this stream wrote is visible to the peers first
        store_release_sys(static_cast<int*>(flags.ptr[p]) + rank, e);
        const int* mine = static_cast<const int*>(flags.ptr[rank]) + p;
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        while (load_acquire_sys(mine) < e) {
            // wall-clock limit, checked every 1024 polls, plus an absolute cap on the number of polls
            if ((++spins & 0x3FFu) == 0 && (global_timer_ns() - t0 > timeout_ns || spins >= 0xFFFFF000u)) {
                atomicCAS(&ctrl[1], 0, 1 + p);
                break;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) ctrl[0] = e;
}

__global__ void __launch_bounds__(256)
p2p_reduce_adam_kernel(PeerTable grads, PeerTable params, float* __restrict__ m, float* __restrict__ v,
                       const double* __restrict__ state, const int* __restrict__ ctrl, int64_t lo, int64_t hi,
                       int world, float lr, float b1, float b2, float eps, float gscale) {
    // a barrier that gave up means some rank's gradients may be missing or still changing: touch nothing
    if (ctrl != nullptr && ctrl[1] != 0) return;
    const double bc1 = 1.0 - state[0];
    const double bc2 = 1.0 - state[1];
    const float step_size = (float)((double)lr / bc1);
    const float bc2_sqrt = (float)sqrt(bc2);
    // [lo, hi) in float4 units; m and v are indexed from the start of the slice
    for (int64_t i = lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi;
         i += (int64_t)gridDim.x * blockDim.x) {
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < DL_MAX_PEERS; ++p) {
            if (p < world) {
                const float4 t = static_cast<const float4*>(grads.ptr[p])[i];
                g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
            }
        }
        float4 pp = static_cast<const float4*>(params.ptr[0])[i];  // every rank's copy holds the same bits
        float4 mm = reinterpret_cast<float4*>(m)[i - lo], vv = reinterpret_cast<float4*>(v)[i - lo];
        pp.x = adam_update(pp.x, g.x, gscale, mm.x, vv.x, step_size, bc2_sqrt, b1, b2, eps);
        pp.y = adam_update(pp.y, g.y, gscale, mm.y, vv.y, step_size, bc2_sqrt, b1, b2, eps);
        pp.z = adam_update(pp.z, g.z, gscale, mm.z, vv.z, step_size, bc2_sqrt, b1, b2, eps);
        pp.w = adam_update(pp.w, g.w, gscale, mm.w, vv.w, step_size, bc2_sqrt, b1, b2, eps);
        reinterpret_cast<float4*>(m)[i - lo] = mm;
        reinterpret_cast<float4*>(v)[i - lo] = vv;
#pragma unroll
        for (int p = 0; p < DL_MAX_PEERS; ++p)
            if (p < world) static_cast<float4*>(params.ptr[p])[i] = pp;
    }
}

__global__ void adam_state_advance_kernel(double* state, const int* __restrict__ ctrl, double b1, double b2) {
    if (ctrl != nullptr && ctrl[1] != 0) return;
    state[0] *= b1;
    state[1] *= b2;
}

// ------------------------------------------------------------------------------------------
// one kernel per exchange: arrive -> reduce + Adam + broadcast -> done
// ------------------------------------------------------------------------------------------
//
// flags of rank q: int32 [DL_P2P_CHANNELS][2][DL_MAX_PEERS]; entry [ch][0][p] is the epoch in which rank p's
// gradients of channel ch became complete ("arrive"), [ch][1][p] the epoch in which rank p finished reading
// everybody's gradients and storing its parameter slice everywhere ("done").  Slot p is written by rank p
// only.  ctrl (local): [0] = status (0 = fine, else 1 + the first peer a bounded wait gave up on; sticky),
// [1 + 2 ch] = epoch of channel ch, [2 + 2 ch] = number of CTAs of the running launch that have finished.
//
// Every CTA waits for the arrive flags itself (they live in this GPU's memory, so polling is local); no CTA
// waits for another CTA of the grid, so the grid need not be resident at once and may share the GPU with
// the backward kernels of the layers below.  The CTA that finishes last publishes "done" to the peers,
// waits for theirs and only then lets the kernel end: whatever follows it in stream order sees every rank's
// parameter stores, and no rank overwrites its gradients while another still reads them.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, uint64_t timeout_ns) {
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (load_acquire_sys(flag) < epoch) {
        // wall-clock limit, checked every 1024 polls, plus an absolute cap on the number of polls
        if ((++spins & 0x3FFu) == 0 && (global_timer_ns() - t0 > timeout_ns || spins >= 0xFFFFF000u)) return false;
    }
    return true;
}

struct ExchangeCtl {       // what the head of an exchange kernel hands to its body and tail
    int epoch;
    bool ok;
};

// Arrive: CTA 0 publishes this rank's arrival to every peer; every CTA waits until all peers have arrived.
__device__ __forceinline__ ExchangeCtl exchange_head(const PeerTable& flags, int* __restrict__ own_flags,
                                                     int* __restrict__ ctrl, int ch, int rank, int world,
                                                     uint64_t timeout_ns) {
    ExchangeCtl c;
    c.ok = ctrl[0] == 0;  // an earlier wait gave up: the state is invalid until the host has looked at it
    // read before any CTA can finish: the epoch word is advanced by the LAST CTA to finish
    c.epoch = ctrl[1 + 2 * ch] + 1;
    if (!c.ok) return c;
    const int arrive = (ch * 2 + 0) * DL_MAX_PEERS;
    bool ok = true;
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        if (blockIdx.x == 0) {
            __threadfence_system();  // the gradients earlier kernels of this GPU wrote are visible to the peers first
            store_release_sys(static_cast<int*>(flags.ptr[p]) + arrive + rank, c.epoch);
        }
        if (!wait_flag(own_flags + arrive + p, c.epoch, timeout_ns)) {
            atomicCAS(&ctrl[0], 0, 1 + p);
            ok = false;
        }
    }
    c.ok = __syncthreads_and(ok);
    return c;
}

// Done: the CTA that finishes last tells the peers, waits for theirs, then advances the epoch (and, on the
// step's last exchange, the optimiser state).
__device__ __forceinline__ void exchange_tail(const PeerTable& flags, int* __restrict__ own_flags,
                                              int* __restrict__ ctrl, double* __restrict__ state, int ch, int rank,
                                              int world, int epoch, int advance, bool wait_peers, float b1, float b2,
                                              uint64_t timeout_ns) {
    __shared__ int last_cta;
    int* const my_done = ctrl + 2 + 2 * ch;
    __syncthreads();  // every thread's parameter stores are ordered before thread 0's fence
    if (threadIdx.x == 0) {
        __threadfence_system();
        last_cta = atomicAdd(my_done, 1) == (int)gridDim.x - 1;
    }
    __syncthreads();
    if (!last_cta) return;
    __threadfence_system();  // the other CTAs' stores, observed through the counter, before the flag below
    const int done = (ch * 2 + 1) * DL_MAX_PEERS;
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        store_release_sys(static_cast<int*>(flags.ptr[p]) + done + rank, epoch);
        // without the wait the caller runs dl_p2p_wait_done before anything reads the parameters or
        // overwrites the gradients: the second rendezvous then costs nothing on the step's critical path
        if (wait_peers && !wait_flag(own_flags + done + p, epoch, timeout_ns)) atomicCAS(&ctrl[0], 0, 1 + p);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        *my_done = 0;
        ctrl[1 + 2 * ch] = epoch;
        if (advance) {
            state[0] *= (double)b1;
            state[1] *= (double)b2;
        }
    }
}

// Bias corrections of THIS step: state holds beta^(t-1) until the step's last exchange advances it (the
// products are rounded on their own, as the stored state of the next step will be: no fused multiply-add).
__device__ __forceinline__ void exchange_step_sizes(const double* __restrict__ state, float lr, float b1, float b2,
                                                    float& step_size, float& bc2_sqrt) {
    const double bc1 = 1.0 - __dmul_rn(state[0], (double)b1);
    const double bc2 = 1.0 - __dmul_rn(state[1], (double)b2);
    step_size = (float)((double)lr / bc1);
    bc2_sqrt = (float)sqrt(bc2);
}

// Second half of a deferred rendezvous: wait until every peer has published "done" for the channel's latest epoch.
__global__ void p2p_wait_done_kernel(const int* __restrict__ own_flags, int* __restrict__ ctrl, int ch, int world,
                                     uint64_t timeout_ns) {
    if (ctrl[0] != 0) return;
    const int epoch = ctrl[1 + 2 * ch];
    const int p = threadIdx.x;
    if (p < world && !wait_flag(own_flags + (ch * 2 + 1) * DL_MAX_PEERS + p, epoch, timeout_ns))
        atomicCAS(&ctrl[0], 0, 1 + p);
}

// For an exchange that has the GPU to itself: 256-thread CTAs, two 16-byte pieces per thread and iteration
// (several peer loads in flight per thread).  [lo, hi) in float4 units of the flat vector; this rank's moments
// of the slice start at mlo.
__global__ void __launch_bounds__(256, 2)
p2p_exchange_adam_kernel(PeerTable grads, PeerTable params, PeerTable flags, int* __restrict__ own_flags,
                         const float4* __restrict__ own_params, float4* __restrict__ m, float4* __restrict__ v,
                         double* __restrict__ state, int* __restrict__ ctrl, int64_t lo, int64_t hi, int64_t mlo,
                         int ch, int advance, int wait_peers, int rank, int world, float lr, float b1, float b2,
                         float eps, float gscale, uint64_t timeout_ns) {
    const ExchangeCtl c = exchange_head(flags, own_flags, ctrl, ch, rank, world, timeout_ns);
    if (!c.ok) return;  // parameters, moments and optimiser state stay untouched
    float step_size, bc2_sqrt;
    exchange_step_sizes(state, lr, b1, b2, step_size, bc2_sqrt);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i0 = lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < hi; i0 += 2 * stride) {
        const int64_t i1 = i0 + stride;
        const bool two = i1 < hi;
        float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
#pragma unroll
        for (int p = 0; p < DL_MAX_PEERS; ++p) {
            if (p < world) {  // rank order: every rank forms the same sum, bit for bit
                const float4 t0 = __ldcg(static_cast<const float4*>(grads.ptr[p]) + i0);
                const float4 t1 = two ? __ldcg(static_cast<const float4*>(grads.ptr[p]) + i1) : make_float4(0.f, 0.f, 0.f, 0.f);
                g0.x += t0.x; g0.y += t0.y; g0.z += t0.z; g0.w += t0.w;
                g1.x += t1.x; g1.y += t1.y; g1.z += t1.z; g1.w += t1.w;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (h == 1 && !two) break;
            const int64_t i = h == 0 ? i0 : i1;
            const float4 g = h == 0 ? g0 : g1;
            float4 pp = own_params[i];  // every rank's copy holds the same bits
            float4 mm = m[mlo + i - lo], vv = v[mlo + i - lo];
            pp.x = adam_update(pp.x, g.x, gscale, mm.x, vv.x, step_size, bc2_sqrt, b1, b2, eps);
            pp.y = adam_update(pp.y, g.y, gscale, mm.y, vv.y, step_size, bc2_sqrt, b1, b2, eps);
            pp.z = adam_update(pp.z, g.z, gscale, mm.z, vv.z, step_size, bc2_sqrt, b1, b2, eps);
            pp.w = adam_update(pp.w, g.w, gscale, mm.w, vv.w, step_size, bc2_sqrt, b1, b2, eps);
            m[mlo + i - lo] = mm;
            v[mlo + i - lo] = vv;
#pragma unroll
            for (int p = 0; p < DL_MAX_PEERS; ++p)
                if (p < world) static_cast<float4*>(params.ptr[p])[i] = pp;
        }
    }
    exchange_tail(flags, own_flags, ctrl, state, ch, rank, world, c.epoch, advance, wait_peers != 0, b1, b2, timeout_ns);
}

// For an exchange that runs while a fused backward kernel fills the GPU from another stream.  Five resident
// CTAs of that kernel (20 warps of 96 registers) leave 1024 registers free in each of an SM's four register
// partitions: one warp of at most 32 registers per partition.  This variant is built for exactly that hole
// (four warps, 32 registers, no shared-memory arrays), so its CTAs are scheduled beside the backward kernel
// instead of after it.  It works on single floats, four per thread and iteration, a warp always on 128
// consecutive bytes.  [lo, hi) and mlo in floats here.
__global__ void __launch_bounds__(128, 16)
p2p_exchange_adam_lean_kernel(PeerTable grads, PeerTable params, PeerTable flags, int* __restrict__ own_flags,
                              const float* __restrict__ own_params, float* __restrict__ m, float* __restrict__ v,
                              double* __restrict__ state, int* __restrict__ ctrl, int64_t lo, int64_t hi,
                              int64_t mlo, int ch, int advance, int wait_peers, int rank, int world, float lr, float b1,
                              float b2, float eps, float gscale, uint64_t timeout_ns) {
    const ExchangeCtl c = exchange_head(flags, own_flags, ctrl, ch, rank, world, timeout_ns);
    if (!c.ok) return;
    float step_size, bc2_sqrt;
    exchange_step_sizes(state, lr, b1, b2, step_size, bc2_sqrt);
    const int64_t stride = (int64_t)gridDim.x * 128 * 4;
    for (int64_t base = lo + (int64_t)blockIdx.x * 128 * 4 + threadIdx.x; base < hi; base += stride) {
        float g[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int p = 0; p < DL_MAX_PEERS; ++p) {
            if (p < world) {  // rank order: every rank forms the same sum, bit for bit
                const float* src = static_cast<const float*>(grads.ptr[p]);
                float t[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) t[k] = base + k * 128 < hi ? __ldcg(src + base + k * 128) : 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) g[k] += t[k];
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t i = base + k * 128;
            if (i >= hi) break;
            float mm = m[mlo + i - lo], vv = v[mlo + i - lo];
            const float pp = adam_update(own_params[i], g[k], gscale, mm, vv, step_size, bc2_sqrt, b1, b2, eps);
            m[mlo + i - lo] = mm;
            v[mlo + i - lo] = vv;
#pragma unroll
            for (int p = 0; p < DL_MAX_PEERS; ++p)
                if (p < world) static_cast<float*>(params.ptr[p])[i] = pp;
        }
    }
    exchange_tail(flags, own_flags, ctrl, state, ch, rank, world, c.epoch, advance, wait_peers != 0, b1, b2, timeout_ns);
}

int fill_table(PeerTable& t, const void* const* host_ptrs, int64_t world) {
    for (int p = 0; p < DL_MAX_PEERS; ++p) t.ptr[p] = nullptr;
    for (int64_t p = 0; p < world; ++p) {
        if (host_ptrs[p] == nullptr) return DL_ERR_ARG;
        t.ptr[p] = const_cast<void*>(host_ptrs[p]);
    }
    return DL_OK;
}

}  // namespace

DL_EXPORT int dl_p2p_enable_peer(int64_t peer_device) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return DL_ERR_LAUNCH;
    if (peer_device == dev) return DL_OK;
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, dev, (int)peer_device) != cudaSuccess || !can) return DL_ERR_UNSUPPORTED;
    const cudaError_t rc = cudaDeviceEnablePeerAccess((int)peer_device, 0);
    if (rc == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();  // clear the sticky-free error state
        return DL_OK;
    }
    return rc == cudaSuccess ? DL_OK : DL_ERR_LAUNCH;
}

DL_EXPORT int dl_p2p_barrier(const void* const* peer_flags_host, int64_t rank, int64_t world, int32_t* ctrl,
                             int64_t timeout_ms, dl_stream_t stream) {
    DL_REQUIRE(peer_flags_host && ctrl && world >= 1 && world <= DL_MAX_PEERS && rank >= 0 && rank < world);
    DL_REQUIRE(timeout_ms > 0 && timeout_ms <= 60000);
    PeerTable flags;
    const int rc = fill_table(flags, peer_flags_host, world);
    if (rc != DL_OK) return rc;
    p2p_barrier_kernel<<<1, 32, 0, dl_cast(stream)>>>(flags, (int)rank, (int)world, ctrl,
                                                     (uint64_t)timeout_ms * 1000000ull);
    return dl_launch_status();
}

DL_EXPORT int dl_p2p_reduce_adam(const void* const* peer_grads_host, const void* const* peer_params_host, float* m,
                                 float* v, double* state, const int32_t* ctrl, int64_t count, int64_t rank,
                                 int64_t world, float lr, float beta1, float beta2, float eps, float gscale,
                                 dl_stream_t stream) {
    DL_REQUIRE(peer_grads_host && peer_params_host && m && v && state && count > 0);
    DL_REQUIRE(world >= 1 && world <= DL_MAX_PEERS && rank >= 0 && rank < world);
    DL_REQUIRE(count % (4 * world) == 0);  // equal slices of whole float4s: the caller pads the flat vector
    PeerTable grads, params;
    int rc = fill_table(grads, peer_grads_host, world);
    if (rc != DL_OK) return rc;
    rc = fill_table(params, peer_params_host, world);
    if (rc != DL_OK) return rc;
    for (int64_t p = 0; p < world; ++p) {
        DL_REQUIRE_ALIGNED(grads.ptr[p], 16);
        DL_REQUIRE_ALIGNED(params.ptr[p], 16);
    }
    DL_REQUIRE_ALIGNED(m, 16);
    DL_REQUIRE_ALIGNED(v, 16);
    // the owner's copy is read as "the" parameters: put it first so the read is local
    void* t = params.ptr[0]; params.ptr[0] = params.ptr[rank]; params.ptr[rank] = t;
    const int64_t quads = count / 4, per = quads / world;
    const int64_t lo = rank * per, hi = lo + per;
    adam_state_advance_kernel<<<1, 1, 0, dl_cast(stream)>>>(state, ctrl, (double)beta1, (double)beta2);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    const int64_t blocks = dl_min64(dl_ceil_div(per, 256), (int64_t)DL_NUM_SMS * 4);
    p2p_reduce_adam_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(grads, params, m, v, state, ctrl, lo, hi,
                                                                       (int)world, lr, beta1, beta2, eps, gscale);
    return dl_launch_status();
}

// DIFFLUT_PEER_BLOCKS=k caps the grid of the whole-vector exchange kernel (a measurement aid: fewer CTAs walk the
// slice in several iterations, so that one iteration's stores overlap the next one's loads).
static int64_t exchange_blocks_override() {
    static const int64_t v = [] {
        const char* e = getenv("DIFFLUT_PEER_BLOCKS");
        return e ? (int64_t)atoi(e) : (int64_t)0;
    }();
    return v;
}

DL_EXPORT int dl_p2p_exchange_adam(const void* const* peer_grads_host, const void* const* peer_params_host,
                                   const void* const* peer_flags_host, float* m, float* v, double* state,
                                   int32_t* ctrl, int64_t offset, int64_t count, int64_t channel, int64_t advance_state,
                                   int64_t overlapped, int64_t defer_done, int64_t rank, int64_t world, float lr,
                                   float beta1, float beta2, float eps, float gscale, int64_t timeout_ms,
                                   dl_stream_t stream) {
    DL_REQUIRE(peer_grads_host && peer_params_host && peer_flags_host && m && v && state && ctrl);
    DL_REQUIRE(world >= 1 && world <= DL_MAX_PEERS && rank >= 0 && rank < world);
    DL_REQUIRE(channel >= 0 && channel < DL_P2P_CHANNELS && timeout_ms > 0 && timeout_ms <= 60000);
    // the slice and every rank's share of it are whole float4s: the caller pads the flat vector
    DL_REQUIRE(count > 0 && offset >= 0 && count % (4 * world) == 0 && offset % (4 * world) == 0);
    PeerTable grads, params, flags;
    int rc = fill_table(grads, peer_grads_host, world);
    if (rc != DL_OK) return rc;
    rc = fill_table(params, peer_params_host, world);
    if (rc != DL_OK) return rc;
    rc = fill_table(flags, peer_flags_host, world);
    if (rc != DL_OK) return rc;
    for (int64_t p = 0; p < world; ++p) {
        DL_REQUIRE_ALIGNED(grads.ptr[p], 16);
        DL_REQUIRE_ALIGNED(params.ptr[p], 16);
        DL_REQUIRE_ALIGNED(flags.ptr[p], 4);
    }
    DL_REQUIRE_ALIGNED(m, 16);
    DL_REQUIRE_ALIGNED(v, 16);
    const int64_t per = count / 4 / world;           // float4s this rank owns of the slice
    const int64_t lo = offset / 4 + rank * per;
    const int64_t mlo = offset / 4 / world;          // the moments hold only this rank's share of every slice
    const uint64_t timeout_ns = (uint64_t)timeout_ms * 1000000ull;
    int* own_flags = static_cast<int*>(flags.ptr[rank]);
    if (overlapped) {
        // one four-warp CTA per SM, beside the resident CTAs of a backward kernel on the caller's other stream
        int64_t blocks = dl_min64(dl_ceil_div(per * 4, 128 * 4), (int64_t)DL_NUM_SMS);
        if (blocks < 1) blocks = 1;
        p2p_exchange_adam_lean_kernel<<<(unsigned)blocks, 128, 0, dl_cast(stream)>>>(
            grads, params, flags, own_flags, static_cast<const float*>(params.ptr[rank]), m, v, state, ctrl, lo * 4,
            (lo + per) * 4, mlo * 4, (int)channel, advance_state != 0, defer_done == 0, (int)rank, (int)world, lr, beta1,
            beta2, eps, gscale, timeout_ns);
    } else {
        int64_t blocks = dl_min64(dl_ceil_div(per, 256 * 2), (int64_t)DL_NUM_SMS * 2);
        if (exchange_blocks_override() > 0) blocks = dl_min64(blocks, exchange_blocks_override());
        if (blocks < 1) blocks = 1;
        p2p_exchange_adam_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(
            grads, params, flags, own_flags, static_cast<const float4*>(params.ptr[rank]),
            reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v), state, ctrl, lo, lo + per, mlo, (int)channel,
            advance_state != 0, defer_done == 0, (int)rank, (int)world, lr, beta1, beta2, eps, gscale, timeout_ns);
    }
    return dl_launch_status();
}

DL_EXPORT int dl_p2p_wait_done(const void* const* peer_flags_host, int32_t* ctrl, int64_t channel, int64_t rank,
                               int64_t world, int64_t timeout_ms, dl_stream_t stream) {
    DL_REQUIRE(peer_flags_host && ctrl && world >= 1 && world <= DL_MAX_PEERS && rank >= 0 && rank < world);
    DL_REQUIRE(channel >= 0 && channel < DL_P2P_CHANNELS && timeout_ms > 0 && timeout_ms <= 60000);
    DL_REQUIRE(peer_flags_host[rank] != nullptr);
    p2p_wait_done_kernel<<<1, 32, 0, dl_cast(stream)>>>(static_cast<const int*>(peer_flags_host[rank]), ctrl, (int)channel,
                                                       (int)world, (uint64_t)timeout_ms * 1000000ull);
    return dl_launch_status();
}
