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
                       const double* __restrict__ state, int64_t lo, int64_t hi, int world, float lr, float b1,
                       float b2, float eps, float gscale) {
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
        pp.x = adam_update(pp.x, g.x * gscale, mm.x, vv.x, step_size, bc2_sqrt, b1, b2, eps);
        pp.y = adam_update(pp.y, g.y * gscale, mm.y, vv.y, step_size, bc2_sqrt, b1, b2, eps);
        pp.z = adam_update(pp.z, g.z * gscale, mm.z, vv.z, step_size, bc2_sqrt, b1, b2, eps);
        pp.w = adam_update(pp.w, g.w * gscale, mm.w, vv.w, step_size, bc2_sqrt, b1, b2, eps);
        reinterpret_cast<float4*>(m)[i - lo] = mm;
        reinterpret_cast<float4*>(v)[i - lo] = vv;
#pragma unroll
        for (int p = 0; p < DL_MAX_PEERS; ++p)
            if (p < world) static_cast<float4*>(params.ptr[p])[i] = pp;
    }
}

__global__ void adam_state_advance_kernel(double* state, double b1, double b2) {
    state[0] *= b1;
    state[1] *= b2;
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
                                 float* v, double* state, int64_t count, int64_t rank, int64_t world, float lr,
                                 float beta1, float beta2, float eps, float gscale, dl_stream_t stream) {
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
    adam_state_advance_kernel<<<1, 1, 0, dl_cast(stream)>>>(state, (double)beta1, (double)beta2);
    if (cudaPeekAtLastError() != cudaSuccess) return DL_ERR_LAUNCH;
    const int64_t blocks = dl_min64(dl_ceil_div(per, 256), (int64_t)DL_NUM_SMS * 4);
    p2p_reduce_adam_kernel<<<(unsigned)blocks, 256, 0, dl_cast(stream)>>>(grads, params, m, v, state, lo, hi,
                                                                       (int)world, lr, beta1, beta2, eps, gscale);
    return dl_launch_status();
}
