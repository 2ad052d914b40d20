// Cross-GPU hand-off for the sharded decode path: the all-gather of an N-split projection is done by the qmv
// kernel itself (it stores its output tile into every rank's buffer through peer mappings, see QmvArgs::extra),
// and this barrier tells every rank that all tiles of a phase have landed.  One process per GPU; the buffers and
// the flag arrays are plain cudaMalloc memory shared with cudaIpc handles (no multicast objects involved).
// The reference is a single-device library and has no counterpart.
#include "common.cuh"

namespace mtc {
namespace {

constexpr int kMaxPeersB = 8;

struct BarrierArgs {
    uint32_t *peer_flags[kMaxPeersB];   // peer p's flag array (kMaxPeersB words), mapped into this process
    uint32_t *local_flags;              // this rank's own array: word p is written by rank p
    uint32_t *epoch;                    // this rank's barrier counter (the same sequence on every rank)
    uint32_t *status;
    int n_peers, rank;
    uint32_t poll_limit;                // bounded wait: 2^22 polls (a few seconds) unless the context says otherwise
};

// <<<1, 32>>>.  After griddepcontrol.wait the kernels before this one (the stores into the peers' buffers) have
// completed; the flag is written with a system-scope release after a system fence and read with an acquire.
__global__ void peer_barrier_kernel(const BarrierArgs a) {
    const int p = threadIdx.x;
    // Programmatic dependent launch on both sides: this kernel is resident before the projections of the phase have
    // finished and waits for them here; the next phase's kernels may start prefetching their weights now and wait
    // for this kernel before they read activations or store.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t e = *a.epoch + 1u;
    if (p < a.n_peers) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[p] + a.rank), "r"(e) : "memory");
        bool seen = false;
        for (uint32_t i = 0; i < a.poll_limit; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.local_flags + p) : "memory");
            if (static_cast<int32_t>(v - e) >= 0) {
                seen = true;
                break;
            }
            __nanosleep(20);
        }
        if (!seen) atomicCAS(a.status, 0u, 0x601u + static_cast<uint32_t>(p));     // rank p never arrived
    }
    __syncwarp();
    if (p == 0) *a.epoch = e;
}

}  // namespace

cudaError_t launch_peer_barrier(Ctx *ctx, cudaStream_t st, uint32_t *const *peer_flags, int n_peers, int rank,
                                uint32_t *local_flags, uint32_t *epoch) {
    if (n_peers < 1 || n_peers > kMaxPeersB || rank < 0 || rank >= n_peers || !peer_flags || !local_flags || !epoch)
        return cudaErrorInvalidValue;
    BarrierArgs a{};
    for (int p = 0; p < n_peers; ++p) {
        if (!peer_flags[p]) return cudaErrorInvalidValue;
        a.peer_flags[p] = peer_flags[p];
    }
    a.local_flags = local_flags;
    a.epoch = epoch;
    a.status = ctx->d_status;
    a.n_peers = n_peers;
    a.rank = rank;
    a.poll_limit = ctx->peer_poll_limit;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, peer_barrier_kernel, a);
}

}  // namespace mtc
