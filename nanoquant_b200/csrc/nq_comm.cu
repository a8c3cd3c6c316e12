// All-gather of the tensor-parallel output shards over peer memory (NVLink), as one small kernel that can
// be captured in a CUDA graph together with the GEMV / GEMM launches.
//
// Every rank owns a buffer at the same layout (symmetric memory; the caller passes every rank's base
// pointer): a flag word per rank and the gathered regions [rank][shard].  A launch
//   1. copies this rank's shard into slot `rank` of the region in EVERY rank's buffer (plain 16-byte peer
//      stores: no TMA, no multicast, no multimem);
//   2. when all its CTAs have done so, signals every peer (system-scope release store of the launch's
//      epoch into word `rank` of the peer's flag array);
//   3. waits - bounded - until its own flag array shows this epoch for every rank: when the kernel has
//      completed, every shard has landed in this rank's region, and stream order does the rest.
// Ranks are separate processes on separate GPUs; a rank can run at most one launch ahead of a peer (its
// wait needs the peer's signal of the same epoch), so consecutive launches must use different regions.
// The epoch is the launch count of the local state (nq_common.cuh: a counter advanced by a fixed span per
// launch), which makes graph replays work.  No counterpart in the reference, which has no distributed code.
#include "nq_common.cuh"

namespace nq {

constexpr int kPushThreads = 256;
constexpr int kMaxPeers = 8;

struct PushParams {
    const uint4* shard;
    size_t n16;                       // 16-byte words of the shard
    char* region[kMaxPeers];          // every rank's gathered region (slot r at r * 16 * n16)
    unsigned* flags[kMaxPeers];       // every rank's flag array (world words)
    unsigned long long* counter;      // local: launch counter
    unsigned* done;                   // local: CTAs that have copied their part (wraps to 0)
    unsigned* status;                 // local: status word
    unsigned spin_limit;              // polls before the wait for a peer gives up
    int world, rank;
};

__global__ void __launch_bounds__(kPushThreads) allgather_push_kernel(const __grid_constant__ PushParams P) {
    __shared__ int is_last;
    // Programmatic dependent launch on both sides (no-ops without the launch attribute): the next kernel of the
    // stream may start its prologue now (it reads the gathered region only behind its own dependency wait, i.e.
    // after this grid has completed), and this grid may have started while the kernel that produces the shard
    // was still running: nothing of the shard is read before the wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // epoch of this launch: every thread reads before the CTA barrier, one thread arrives behind it
    unsigned long long c;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(P.counter) : "memory");
    const unsigned epoch = (unsigned)(c / kTagSpan) + 1u;
    __syncthreads();
    if (threadIdx.x == 0) launch_arrive(P.counter, blockIdx.x == 0, gridDim.x);
    // 1. this rank's shard into slot `rank` of every rank's region
    const size_t stride = (size_t)gridDim.x * kPushThreads;
    for (size_t i = (size_t)blockIdx.x * kPushThreads + threadIdx.x; i < P.n16; i += stride) {
        const uint4 v = P.shard[i];
        for (int p = 0; p < P.world; ++p)
            reinterpret_cast<uint4*>(P.region[p] + (size_t)P.rank * 16 * P.n16)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicInc(P.done, gridDim.x - 1) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    // 2. all CTAs have stored and fenced: tell every peer, 3. wait for every peer
    __threadfence_system();
    if ((int)threadIdx.x < P.world) {
        unsigned* dst = P.flags[threadIdx.x] + P.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
        const unsigned* mine = P.flags[P.rank] + threadIdx.x;
        // An earlier launch on this state that gave up has left its mark: a peer is missing or late, and every
        // later gather of a replayed step would wait its full limit again.  Such launches poll once and go on.
        unsigned st0;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(st0) : "l"(P.status) : "memory");
        const unsigned limit = st0 ? 0u : P.spin_limit;
        for (unsigned spins = 0;; ++spins) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int)(v - epoch) >= 0) break;
            if (spins >= limit) {
                atomicExch(P.status, (unsigned)(-NQ_ERR_TIMEOUT));
                break;
            }
            __nanosleep(64);
        }
    }
}

static unsigned g_push_limit = kSpinLimit;

}  // namespace nq

using namespace nq;

extern "C" {

size_t nq_allgather_state_bytes(void) { return 64; }
size_t nq_allgather_flags_bytes(int world) { return world > 0 && world <= kMaxPeers ? 256 : 0; }

int nq_allgather_push(const void* shard, size_t shard_bytes, void* const* rank_bases_host, size_t flags_offset,
                      size_t region_offset, void* local_state, int world, int rank, nq_stream_t stream) {
    if (!shard || !rank_bases_host || !local_state) return NQ_ERR_NULL;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return NQ_ERR_SHAPE;
    if (shard_bytes == 0 || shard_bytes % 16 || flags_offset % 16 || region_offset % 16) return NQ_ERR_ALIGN;
    if (!aligned16(shard) || !aligned16(local_state)) return NQ_ERR_ALIGN;
    PushParams P;
    P.shard = static_cast<const uint4*>(shard);
    P.n16 = shard_bytes / 16;
    for (int p = 0; p < kMaxPeers; ++p) {
        char* base = p < world ? static_cast<char*>(rank_bases_host[p]) : nullptr;
        if (p < world && (!base || !aligned16(base))) return NQ_ERR_ALIGN;
        P.region[p] = base ? base + region_offset : nullptr;
        P.flags[p] = base ? reinterpret_cast<unsigned*>(base + flags_offset) : nullptr;
    }
    P.counter = static_cast<unsigned long long*>(local_state);
    P.done = static_cast<unsigned*>(local_state) + 2;
    P.status = static_cast<unsigned*>(local_state) + 3;
    P.spin_limit = g_push_limit;
    P.world = world;
    P.rank = rank;
    size_t ctas = (P.n16 + (size_t)kPushThreads * 4 - 1) / ((size_t)kPushThreads * 4);   // four words per thread
    const size_t cap = (size_t)sm_count();
    ctas = ctas < 1 ? 1 : (ctas > cap ? cap : ctas);
    // programmatic stream serialization: see the kernel; plain launches from then on if the driver refuses it once
    static bool pdl_ok = true;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kPushThreads);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl_ok ? 1 : 0;
    void* args[] = {&P};
    cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)allgather_push_kernel, args);
    if (e != cudaSuccess && pdl_ok) {
        (void)cudaGetLastError();
        pdl_ok = false;
        cfg.numAttrs = 0;
        e = cudaLaunchKernelExC(&cfg, (const void*)allgather_push_kernel, args);
    }
    NQ_CUDA_TRY(e);
    return NQ_OK;
}

unsigned nq_allgather_set_wait_limit(unsigned polls) {
    const unsigned old = g_push_limit;
    g_push_limit = polls ? polls : kSpinLimit;
    return old;
}

int nq_allgather_status(const void* local_state, nq_stream_t stream) {
    if (!local_state) return NQ_ERR_NULL;
    unsigned h[4] = {0, 0, 0, 0};
    NQ_CUDA_TRY(cudaMemcpyAsync(h, local_state, sizeof(h), cudaMemcpyDeviceToHost, as_stream(stream)));
    NQ_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    return h[3] == 0 ? NQ_OK : -(int)h[3];
}

}  // extern "C"
