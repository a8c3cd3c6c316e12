// Prefill GEMM for the binary low-rank linear on the 5th-generation tensor cores.
//
//   stage 1:  t[T, R] = ((x * s_in) . V^T) * s_mid        (t kept in the I/O dtype by default)
//   stage 2:  y[T, M] = (t . U^T) * s_out
//
// Each stage is one launch of the same kernel: Out[T, Nout] = (A[T, K] . W[Nout, K]^T) * post,
// where W = +-pre[k] comes from packed sign bits.  One CTA computes a (128 or 256)-token x
// (128 or 256)-row output tile (or its share of K, see split-K below):
//
//   warp 0      TMA producer: the activation tile [128|256 tokens x 64 k] through a tensor map
//               (cp.async.bulk.tensor, 128-byte swizzle), one per k block.
//   warp 2      the packed sign bits of the tile's weight rows (1-D bulk copies of the GEMV tile
//               layout) and the input scales, one 256-column chunk per step, ahead of the expand warps.
//               (One loading thread for both was measured 10 % slower, an idle warp 5 % slower.)
//   warp 1      one thread issues tcgen05.mma (M = 128 tokens, N = 128|256 rows, K = 16, kind::f16,
//               fp32 accumulator in tensor memory) and commits the stage's buffers back with
//               tcgen05.commit.  The tiles smaller than 256 x 256 have a second issuer (warp 3) with
//               an accumulator of its own on the odd k blocks.
//   then 8|16   expand warps turn the bits into +-pre[k] bf16/fp16 directly in the K-major
//               128-byte-swizzled layout the MMA reads (the product x * (+-s_in) is then exact
//               inside the MMA; pre-scaling x would round it), fence.proxy.async, arrive on the
//               stage's "ready" barrier; afterwards the same warps run the epilogue.
//   epilogue    tcgen05.ld of the accumulator(s) (lane = token, column = output row),
//               * post[n], saturate, convert, 16-byte stores.
//
// Launches with fewer output tiles than SMs split K: over independent CTAs with fp32 slabs in global
// memory and a last-CTA reduction (up to 24 tokens), or over the CTAs of a thread-block cluster that
// exchange their partial sums through distributed shared memory (more tokens); see GemmParams::csplit
// and plan_group.  bf16 linears may keep their intermediate as fp16 times a per-token power of two
// (row_bound_kernel, nq_gemm_set_precise_intermediate).
//
// The packed operand is the same tile layout the decode GEMV streams (nq_rows_to_tiles),
// so a layer keeps one copy of its weights for both kernels.  No TMA multicast is used.
// Every mbarrier wait is bounded; on expiry a status word is set, the CTA drains and
// frees its tensor memory.
//
// replaces: src/nanoquant/kernel/cuda/gemm_kernel.cu:278-791 (Marlin-derived mma.sync
// kernel with register-level dequantisation) and src/nanoquant/kernel/cuda/gemm.cpp:59-122
// of the reference.
#include <cuda.h>

#include <cstdlib>
#include <cstring>

#include "nq_common.cuh"

namespace nq {

constexpr int kBM = 128;            // tokens per MMA (MMA M, tensor-memory lanes)
constexpr int kBK = 64;             // k per pipeline stage: 128 bytes of bf16 = one swizzle row
constexpr int kGroupThreads = 256;                          // expand threads that share one k block
constexpr int kTileBytes = kBM * kBK * 2;          // 16 KB: one 128-row operand tile
constexpr int kPreBytes = 256 * 2;                 // input scales of one 256-column chunk
constexpr unsigned kWaitLimit = 1u << 21;   // attempts of up to ~2 us each

// Tile configuration: MH x 128 tokens by NH x 128 weight rows per CTA.  One expanded weight
// tile feeds MH MMAs and one activation tile meets 128 * NH weight rows, which sets the
// expansion work and the L2 traffic per MAC.  Shared memory map: offsets from a
// 1024-byte aligned base.
template <int MH, int NH>
struct GemmCfg {
    static constexpr int kStages = (MH * NH == 4) ? 3 : (MH * NH == 2 ? 4 : 6);
    static constexpr int kBN = 128 * NH;                    // MMA N, tensor-memory columns per accumulator
    static constexpr int kABytes = MH * kTileBytes;
    static constexpr int kWBytes = NH * kTileBytes;
    static constexpr int kBitsSlotBytes = (kBN / 16) * 512; // row groups x one 256-column chunk of sign bits
    // chunks of sign bits in flight (a power of two): they come from HBM, and with the small tiles, whose
    // k blocks are short, two slots cover less than the memory latency
    static constexpr int kBitsSlots = (NH == 2) ? 2 : 4;
    static constexpr int kOffA = 0;
    static constexpr int kOffW = kOffA + kStages * kABytes;
    static constexpr int kOffBits = kOffW + kStages * kWBytes;
    static constexpr int kOffPre = kOffBits + kBitsSlots * kBitsSlotBytes;   // input scales of a chunk, beside its bits
    static constexpr int kOffBar = kOffPre + kBitsSlots * kPreBytes;
    static constexpr int kNumBars = 2 * kStages + 2 * kBitsSlots + 1;  // ready, free, bits_full, bits_empty, accum
    static constexpr int kOffMisc = kOffBar + kNumBars * 8;   // tmem base address, abort flag
    static constexpr int kOffPost = (kOffMisc + 16 + 15) & ~15;   // output scales of the tile as fp32 (read as float4)
    static_assert(kOffPost % 16 == 0 && kOffBar % 8 == 0 && kOffBits % 16 == 0 && kOffPre % 16 == 0, "shared memory map alignment");
    static constexpr int kOffBias = kOffPost + kBN * 4;            // bias of the tile as fp32
    static constexpr int kSmemBytes = kOffBias + kBN * 4 + 1024;   // + slack for the 1024-byte alignment
    // MMA-issuing threads.  The small tiles are bound by the issuing thread (waits and instruction issue cost
    // more cycles than their MMAs take), so two threads take alternate k blocks, each into an accumulator of
    // its own, and the epilogue adds the two.  The 256 x 256 tile is bound by the tensor pipe and fills the
    // tensor memory with one accumulator set.
    static constexpr int kIssuers = (MH * NH == 4) ? 1 : 2;
    // Expand groups of 256 threads on alternate k blocks: the expansion of a k block is a chain of dependent
    // steps, so the small tiles (short k blocks) need two groups to keep up with two issuers.
    static constexpr int kGroups = (MH * NH == 4) ? 1 : 2;
    static constexpr int kExpandThreads = kGroups * kGroupThreads;
    // warp 0 activation TMA, warp 1 MMA, warp 2 sign bits, warp 3 second MMA issuer (if any), then expand + epilogue
    static constexpr int kFirstExpandWarp = 2 + kIssuers;
    static constexpr int kThreads = 32 * kFirstExpandWarp + kExpandThreads;
    static constexpr int kTmemCols = kIssuers * MH * kBN;
};

// One linear's stage inside a launch.  A launch runs the same stage of up to four linears that share the
// token count (q/k/v, gate/up): their output tiles are laid side by side along grid.x.
struct alignas(64) GemmJob {
    CUtensorMap map_a;     // activations [T, K], box 64 x (128 * MH), 128-byte swizzle
    const uint4* tiles;    // packed weights, GEMV tile layout [row_groups][chunks][32]
    const void* pre;       // [K] input scales (I/O dtype) or nullptr (weights are +-1)
    const void* post;      // [Nout] output scales (I/O dtype) or nullptr
    void* out;             // [T, ld_out] I/O dtype
    const int* row_exp;    // [T] per-token exponents of the intermediate or nullptr (see GemmParams::exp_sign)
    const void* bias;      // [Nout] (I/O dtype) or nullptr, added behind the output scale
    const void* resid;     // [T, ld_res] (I/O dtype) or nullptr, added behind the bias
    long long ld_out, ld_res;
    // split-K (few tokens, few output tiles): `splits` CTAs along grid.z share an output tile, each over
    // `chunks_per` 256-column chunks; partial sums go to fp32 slabs [split][Nout][t_pad] and the CTA that
    // arrives last at the tile's counter adds them up in split order and writes the output.
    float* slabs;
    unsigned* counters;    // one per output tile of this job, zero between launches
    int K, Nout;
    int chunks, row_groups;
    int splits, chunks_per;
    int tile0;             // first grid.x index of this job's tiles
};
constexpr int kMaxGemmJobs = 4;

struct GemmParams {
    GemmJob job[kMaxGemmJobs];
    int njobs;
    unsigned* status;      // device status word (0 = ok)
    int T, t_pad;          // tokens; slab row length (tokens, multiple of 4)
    int is_bf16;           // type of the scales, bias and residual (the I/O type of the linear)
    int a_bf16;            // type of the MMA operands: activations and expanded weights (bf16, else fp16)
    int out_bf16;          // type of the output (bf16, else fp16)
    int saturate;          // apply the reference's output saturation bounds
    // bf16 linears keep their rank-R intermediate as fp16 times a per-token power of two (11 significant bits
    // instead of 8): stage 1 multiplies row t by 2^row_exp[t] (exp_sign = +1), stage 2 by 2^-row_exp[t] (-1).
    // The exponents come from row_bound_kernel; 0: no row scaling.
    int exp_sign;
    // Cluster split-K (more than 24 tokens, fewer output tiles than SMs): the `csplit` CTAs of a thread-block
    // cluster along grid.z share an output tile, each over `chunks_per` 256-column chunks of every job.  After the
    // main loops the accumulators are exchanged through distributed shared memory: 32-column blocks of the tile
    // are dealt round-robin to the CTAs of the cluster, every CTA stores the blocks it does not own into the
    // owner's (by then idle) pipeline buffers, and the owner adds the partial sums in rank order and runs the
    // epilogue of its blocks.  1 = no cluster.
    int csplit;
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One bounded attempt: the hardware suspends the thread until the phase completes or the
// time hint (ns) runs out, so a waiting warp does not compete for issue slots.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(2000u)
        : "memory");
    return ok != 0;
}

// Bounded wait on an mbarrier phase.  Returns false when the limit expired or another
// thread of the CTA already gave up; the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned* status) {
    if (mbar_try(bar, parity)) return true;   // the common case: already complete
    for (unsigned i = 0; i < kWaitLimit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(status, (unsigned)(-NQ_ERR_TIMEOUT));
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);          // start address, LBO = 1 (unused)
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);             // SBO, version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Barrier of the thread-block cluster (every thread of every CTA of the cluster arrives): a hardware barrier
// like __syncthreads(), with release/acquire ordering of the distributed-shared-memory stores before it.
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of this CTA's shared-memory location `local` in the CTA of rank `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ---------------------------------------------------------------------------
// the kernel: one 128 x 128 output tile per CTA
// ---------------------------------------------------------------------------
template <int MH, int NH>
__global__ void __launch_bounds__(GemmCfg<MH, NH>::kThreads) gemm_stage_kernel(const __grid_constant__ GemmParams P) {
    using C = GemmCfg<MH, NH>;
    constexpr int kGemmStages = C::kStages, kBN = C::kBN, kBitsSlotBytes = C::kBitsSlotBytes;
    constexpr int kBitsSlots = C::kBitsSlots, kSlotShift = (kBitsSlots == 4) ? 2 : 1;
    constexpr int kExpandThreads = C::kExpandThreads, kGroups = C::kGroups, kGemmThreads = C::kThreads;
    constexpr int kFirstExpandWarp = C::kFirstExpandWarp;
    constexpr int kOffA = C::kOffA, kOffW = C::kOffW, kOffBits = C::kOffBits, kOffPre = C::kOffPre;
    constexpr int kOffBar = C::kOffBar, kOffMisc = C::kOffMisc, kOffPost = C::kOffPost, kOffBias = C::kOffBias;
    extern __shared__ unsigned char smem_raw[];
    // align inside the shared window (pointer + offset keeps the shared address space visible to the compiler)
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int ji = 0;
    while (ji + 1 < P.njobs && (int)blockIdx.x >= P.job[ji + 1].tile0) ++ji;
    const GemmJob& J = P.job[ji];
    // grid.z is the largest split count of the launch; the CTAs of a cluster all stay (they meet at its barriers)
    if (P.csplit == 1 && (int)blockIdx.z >= J.splits) return;
    const int tile = (int)blockIdx.x - J.tile0;
    const int n0 = tile * kBN;   // first weight row of the tile
    const int m0 = blockIdx.y * (kBM * MH);   // first token of the tile
    // k range of this CTA (all of K unless the launch is split): whole 256-column chunks
    const int c_begin = (int)blockIdx.z * J.chunks_per;
    const int c_end = min(J.chunks, c_begin + J.chunks_per);
    const int kb_begin = 4 * c_begin;
    const int nkb = min((J.K + kBK - 1) / kBK, 4 * c_end) - kb_begin;   // k blocks of this CTA

    // One barrier per stage and direction: "ready" completes when the activation tile has landed (the
    // producer's expect-tx arrival plus the TMA's bytes) AND the expand group has arrived for the weight
    // tile, so the MMA thread waits once per k block; "free" is committed once by the MMA thread and both
    // the producer and the expanders wait on it.
    auto bar_ready = [&](int s) { return sbase + kOffBar + 8 * s; };
    auto bar_free = [&](int s) { return sbase + kOffBar + 8 * (kGemmStages + s); };
    auto bar_bits_full = [&](int b) { return sbase + kOffBar + 8 * (2 * kGemmStages + b); };
    auto bar_bits_empty = [&](int b) { return sbase + kOffBar + 8 * (2 * kGemmStages + kBitsSlots + b); };
    const uint32_t bar_accum = sbase + kOffBar + 8 * (2 * kGemmStages + 2 * kBitsSlots);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffMisc + 4);

    // Programmatic dependent launch: the next kernel of the stream (normally the second stage, or the next
    // linear's first stage) may start its prologue and its weight expansion on SMs this grid leaves idle.
    // It needs no resource of this grid to finish.  In turn this kernel touches memory that an earlier kernel
    // may still use only behind griddepcontrol.wait: the activation loads (warp 0) and the output stores.
    // Weights and scales are constants of the layer.  Both instructions are no-ops without the launch attribute.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 32)   // the activation tile's descriptor on its way while the barriers are set up
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&J.map_a)) : "memory");
    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(bar_ready(s), 1 + kGroupThreads);
            mbar_init(bar_free(s), 1);
        }
        for (int b = 0; b < kBitsSlots; ++b) {
            mbar_init(bar_bits_full(b), 1);
            mbar_init(bar_bits_empty(b), kExpandThreads);
        }
        mbar_init(bar_accum, C::kIssuers);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // input-scale slots start finite: a partial last k block leaves older (finite) values behind
    for (int i = threadIdx.x; i < kBitsSlots * kPreBytes / 4; i += kGemmThreads)
        reinterpret_cast<uint32_t*>(smem + kOffPre)[i] = 0;
    // Output scales and bias of this tile: expand thread i loads those of column i now (the values are needed
    // only in the epilogue, and nothing here waits for them) and puts them into shared memory behind its main loop.
    uint32_t raw_post = 0, raw_bias = 0;
    {
        const int i = (int)threadIdx.x - 32 * kFirstExpandWarp;
        if (i >= 0 && i < kBN && n0 + i < J.Nout) {
            if (J.post) raw_post = 0x10000u | static_cast<const uint16_t*>(J.post)[n0 + i];
            if (J.bias) raw_bias = 0x10000u | static_cast<const uint16_t*>(J.bias)[n0 + i];
        }
    }
    if (warp == 1) {  // tensor-memory allocation: 128 fp32 columns per accumulator, by one whole warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"((uint32_t)C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int nrg = J.row_groups - (n0 >> 4);          // row groups of this tile that exist
    nrg = nrg > kBN / 16 ? kBN / 16 : nrg;

    bool expand_ok = true;   // expand warps: no wait of this thread has expired
    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations come from the previous kernel
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % kGemmStages;
                const uint32_t ph = (kb / kGemmStages) & 1;
                if (!mbar_wait(bar_free(s), ph ^ 1, abort_flag, P.status)) break;
                mbar_expect_tx(bar_ready(s), (uint32_t)(MH * kTileBytes));
                tma_load_2d(sbase + kOffA + s * (C::kABytes), &J.map_a, (kb_begin + kb) * kBK, m0, bar_ready(s));
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ sign bits + input scales, one 256-column
        // chunk per step, running ahead of the expand warps by the two chunk slots
        if (lane == 0) {
            const int nchunks = (nkb + 3) >> 2;
            for (int cl = 0; cl < nchunks; ++cl) {
                const int b = cl & (kBitsSlots - 1), c = c_begin + cl;
                if (!mbar_wait(bar_bits_empty(b), ((cl >> kSlotShift) & 1) ^ 1, abort_flag, P.status)) break;
                int pre_bytes = 0;
                if (J.pre) {
                    const int left = J.K - c * 256;
                    pre_bytes = (left < 256 ? left : 256) * 2;
                }
                mbar_expect_tx(bar_bits_full(b), (uint32_t)nrg * 512u + (uint32_t)pre_bytes);
                for (int rg = 0; rg < nrg; ++rg)
                    bulk_load(sbase + kOffBits + b * kBitsSlotBytes + rg * 512,
                              J.tiles + ((size_t)((n0 >> 4) + rg) * J.chunks + c) * 32, 512u, bar_bits_full(b));
                if (pre_bytes)
                    bulk_load(sbase + kOffPre + b * kPreBytes, static_cast<const char*>(J.pre) + (size_t)c * 512,
                              (uint32_t)pre_bytes, bar_bits_full(b));
            }
        }
    } else if (warp == 1 || (C::kIssuers == 2 && warp == 3)) {
        // ------------------------------------------------------------ MMA issuers
        const int mw = warp == 1 ? 0 : 1;
        if (lane == 0 && mw < C::kIssuers) {
            const uint32_t acc_base = tmem_base + (uint32_t)(mw * MH * kBN);
            const uint32_t fmt = P.a_bf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kBN >> 3) << 17) |
                                   ((uint32_t)(kBM >> 4) << 24);
            bool ok = true;
            for (int kb = mw; kb < nkb && ok; kb += C::kIssuers) {
                const int s = kb % kGemmStages;
                const uint32_t ph = (kb / kGemmStages) & 1;
                ok = mbar_wait(bar_ready(s), ph, abort_flag, P.status);
                if (!ok) break;
                tc_fence_after();
                // descriptors of the stage; inside the 128-byte swizzle row the k offset (32 bytes per MMA) is
                // added to the start-address field (units of 16 bytes)
                const uint64_t a_desc = umma_desc(sbase + kOffA + s * (C::kABytes));
                const uint64_t w_desc = umma_desc(sbase + kOffW + s * C::kWBytes);
#pragma unroll
                for (int mh = 0; mh < MH; ++mh)
#pragma unroll
                    for (int k4 = 0; k4 < kBK / 16; ++k4)
                        umma_f16(acc_base + (uint32_t)(mh * kBN), a_desc + (uint64_t)((mh * kTileBytes + k4 * 32) >> 4),
                                 w_desc + (uint64_t)((k4 * 32) >> 4), idesc, (kb != mw || k4 != 0) ? 1u : 0u);
                umma_commit(bar_free(s));   // the stage's buffers are free once these MMAs have read them
            }
            // arrives when this thread's MMAs are complete (at once if it had no k block)
            if (ok) umma_commit(bar_accum);
        }
    } else {
        // ------------------------------------------------------------ expand warps
        // The expansion of one k block is a chain of dependent steps (wait, shared-memory reads, a few ALU
        // operations, stores, proxy fence, arrive) whose latency, not its instruction count, bounds a
        // group's rate; the small tiles run two groups of eight warps on alternate k blocks.
        const int tu = threadIdx.x - 32 * kFirstExpandWarp;
        const int grp = tu / kGroupThreads, tl = tu % kGroupThreads;
        const uint32_t one2 = P.a_bf16 ? 0x3F803F80u : 0x3C003C00u;
        bool ok = true;
        int c_seen = -1;
        for (int kb = grp; kb < nkb && ok; kb += kGroups) {
            const int s = kb % kGemmStages;
            const uint32_t ph = (kb / kGemmStages) & 1;
            const int c = kb >> 2, b = c & (kBitsSlots - 1), sub = kb & 3;
            if (c != c_seen) { ok = mbar_wait(bar_bits_full(b), (c >> kSlotShift) & 1, abort_flag, P.status); c_seen = c; }
            ok = ok && mbar_wait(bar_free(s), ph ^ 1, abort_flag, P.status);
            if (!ok) break;
            const uint4* bits = reinterpret_cast<const uint4*>(smem + kOffBits + b * kBitsSlotBytes);
            const uint2* pre2 = reinterpret_cast<const uint2*>(smem + kOffPre + b * kPreBytes + sub * (kBK * 2));
            unsigned char* wt = smem + kOffW + s * C::kWBytes;
            // all shared-memory reads of the k block first, then the stores
            uint4 w4[NH];
#pragma unroll
            for (int it = 0; it < NH; ++it) w4[it] = bits[tl + it * kGroupThreads];
            const int l = tl & 31, g = l >> 2, q = l & 3;   // lane of the GEMV tile (same for every task)
            uint2 pp[4];                                      // input scales of columns 32*jj + 16*h + 4q .. +3
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                if (J.pre) pp[c4] = pre2[(32 * (c4 >> 1) + 16 * (c4 & 1) + 4 * q) >> 2];
                else pp[c4] = make_uint2(one2, one2);
            }
#pragma unroll
            for (int it = 0; it < NH; ++it) {
                const int rg = (tl + it * kGroupThreads) >> 5;   // row group of the task
                const uint32_t comp[4] = {w4[it].x, w4[it].y, w4[it].z, w4[it].w};   // {row g h0, row g+8 h0, row g h1, row g+8 h1}
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = 2 * sub + jj;                      // class of the 32 columns
#pragma unroll
                    for (int ci = 0; ci < 4; ++ci) {
                        const int h = ci >> 1, row = 16 * rg + g + 8 * (ci & 1);
                        const uint32_t u = (comp[ci] << (7 - j)) & 0x80808080u;   // bit 8b+j -> sign of byte b
                        const uint32_t v0 = __byte_perm(u, 0u, 0x1404) ^ pp[2 * jj + h].x;   // columns 4q, 4q+1
                        const uint32_t v1 = __byte_perm(u, 0u, 0x3424) ^ pp[2 * jj + h].y;   // columns 4q+2, 4q+3
                        const int c16 = (32 * jj + 16 * h + 4 * q) >> 3;          // 16-byte chunk of the 128-byte row
                        *reinterpret_cast<uint2*>(wt + row * 128 + ((c16 ^ (row & 7)) << 4) + 8 * (q & 1)) =
                            make_uint2(v0, v1);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA
            mbar_arrive(bar_ready(s));
            // this group's last k block of the chunk: release the chunk's bits (both groups arrive, except
            // that a group without a block in a partial last chunk has nothing to release or to wait for)
            if (((kb + kGroups) >> 2) != c || kb + kGroups >= nkb) mbar_arrive(bar_bits_empty(b));
        }
        if (tu < kBN) {
            auto as_float = [&](uint32_t raw, float dflt) {
                if (!(raw & 0x10000u)) return dflt;
                return P.is_bf16 ? __uint_as_float(raw << 16) : __half2float(__ushort_as_half((unsigned short)raw));
            };
            reinterpret_cast<float*>(smem + kOffPost)[tu] = as_float(raw_post, 1.f);
            reinterpret_cast<float*>(smem + kOffBias)[tu] = as_float(raw_bias, 0.f);
        }
        asm volatile("bar.sync 2, %0;" ::"n"(kExpandThreads) : "memory");   // scales visible to every expand thread
        if (ok) ok = mbar_wait(bar_accum, 0, abort_flag, P.status);   // this CTA's MMAs are complete
        expand_ok = ok;
    }
    // ---------------------------------------------------------------- epilogue (expand warps)
    const bool is_expand = warp >= kFirstExpandWarp;
    const int lq = warp & 3;                                   // tensor-memory lane quarter this warp may read
    const int sub_w = (warp - kFirstExpandWarp) >> 2;          // index among the warps of that quarter
    constexpr int kBlocks = MH * (kBN / 32);                   // 128-token x 32-column blocks of the tile
    constexpr int kBlockBytes = 128 * 32 * 4;
    // accumulator block `blk` of this CTA (both issuers' sums) into r; zeros if this CTA had no k block.
    // Warp-collective: every lane of the warp takes part.
    auto load_block = [&](int blk, uint32_t (&r)[32]) {
        const int mh = blk / (kBN / 32), c0 = (blk % (kBN / 32)) * 32;
        __syncwarp();
        if (nkb <= 0) {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = 0u;
            return;
        }
        tmem_ld32(tmem_base + ((uint32_t)(32 * lq) << 16) + (uint32_t)(mh * kBN + c0), r);
        if (C::kIssuers == 2 && nkb > 1) {   // the second issuer's accumulator
            uint32_t r2[32];
            tmem_ld32(tmem_base + ((uint32_t)(32 * lq) << 16) + (uint32_t)(MH * kBN + mh * kBN + c0), r2);
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) + __uint_as_float(r2[e]));
        }
    };
    const int crank = P.csplit > 1 ? (int)blockIdx.z : 0;      // cluster dimensions are (1, 1, csplit)
    const int max_owned = (kBlocks + P.csplit - 1) / P.csplit;
    if (P.csplit > 1) {
        // every CTA of the cluster has finished its main loop: the pipeline buffers (from kOffA) are free to
        // receive the partial sums of the blocks this CTA owns, slot [source rank][block / csplit]; inside a slot
        // [lane quarter][16-byte piece of the 32 columns][lane], so that a warp's store covers 512 contiguous bytes
        // (stores that scatter over 32 rows took 5 us per exchange: the cluster network moves whole lines)
        cluster_sync_all();
        if (is_expand && expand_ok) {
            tc_fence_after();
#pragma unroll 1
            for (int blk = sub_w; blk < kBlocks; blk += kExpandThreads / 128) {
                const int owner = blk % P.csplit;
                if (owner == crank) continue;
                if (m0 + kBM * (blk / (kBN / 32)) + 32 * lq >= P.T) continue;   // none of this warp's 32 tokens exists
                uint32_t r[32];
                load_block(blk, r);
                const uint32_t slot = sbase + kOffA + (uint32_t)((crank * max_owned + blk / P.csplit) * kBlockBytes + lq * 4096 + lane * 16);
                const uint32_t dst = cluster_map(slot, (uint32_t)owner);
#pragma unroll
                for (int c = 0; c < 8; ++c)   // a warp stores 512 contiguous bytes per instruction
                    cluster_store4(dst + (uint32_t)(c * 512), r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
            }
        }
        cluster_sync_all();
    }
    if (is_expand) {
        bool ok = expand_ok;
        // the output buffer may still be read by the kernel before the previous one (its input): the accumulator
        // is complete only after warp 0 passed its wait, but each thread has to order its own stores
        asm volatile("griddepcontrol.wait;" ::: "memory");
        // 32-column blocks of the MH accumulators, dealt round-robin to the warps that share a lane quarter
        if (ok) {
            tc_fence_after();
            const float lim = P.saturate ? (P.out_bf16 ? 3.3895313892515355e+38f : 64504.0f) : 3.4e38f;
            const float4* post4 = reinterpret_cast<const float4*>(smem + kOffPost);
            // per-token power of two of the intermediate (exact: the exponent is an integer), one load per
            // token and thread ahead of the blocks (inside the loop its latency would repeat for every block)
            float rs_mh[MH];
#pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
                const int row = m0 + kBM * mh + 32 * lq + lane;
                rs_mh[mh] = (J.row_exp && row < P.T) ? exp2f((float)(P.exp_sign * J.row_exp[row])) : 1.f;
            }
#pragma unroll 1
            for (int blk = sub_w; blk < kBlocks; blk += kExpandThreads / 128) {
                if (P.csplit > 1 && blk % P.csplit != crank) continue;   // another CTA of the cluster finishes this block
                const int mh = blk / (kBN / 32), c0 = (blk % (kBN / 32)) * 32;
                const int row = m0 + kBM * mh + 32 * lq + lane;     // token
                if (row - lane >= P.T) continue;                     // none of this warp's 32 tokens exists
                uint32_t r[32];
                load_block(blk, r);
                if (P.csplit > 1) {   // the other ranks' partial sums, in rank order
                    for (int rk = 0; rk < P.csplit; ++rk) {
                        if (rk == crank) continue;
                        const unsigned char* src = smem + kOffA + (size_t)(rk * max_owned + blk / P.csplit) * kBlockBytes + lq * 4096 + lane * 16;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const float4 v = *reinterpret_cast<const float4*>(src + c * 512);
                            r[4 * c] = __float_as_uint(__uint_as_float(r[4 * c]) + v.x);
                            r[4 * c + 1] = __float_as_uint(__uint_as_float(r[4 * c + 1]) + v.y);
                            r[4 * c + 2] = __float_as_uint(__uint_as_float(r[4 * c + 2]) + v.z);
                            r[4 * c + 3] = __float_as_uint(__uint_as_float(r[4 * c + 3]) + v.w);
                        }
                    }
                }
                // The tensor-memory loads above are warp-collective: every lane takes part in every round, and a
                // lane without a valid output only skips the stores.
                const bool valid = row < P.T && n0 + c0 < J.Nout;
                const float rs = MH == 1 ? rs_mh[0] : (mh == 0 ? rs_mh[0] : rs_mh[MH - 1]);
                if (J.splits > 1) {   // partial sums of this k range: a warp writes 32 consecutive tokens per column
                    if (valid) {
                        float* slab = J.slabs + ((size_t)blockIdx.z * J.Nout + n0 + c0) * P.t_pad + row;
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if (n0 + c0 + e < J.Nout) slab[(size_t)e * P.t_pad] = __uint_as_float(r[e]);
                    }
                } else if (valid) {
                const float4* bias4 = reinterpret_cast<const float4*>(smem + kOffBias);
                const uint16_t* res_row = J.resid ? static_cast<const uint16_t*>(J.resid) + (size_t)row * J.ld_res + n0 + c0 : nullptr;
                uint32_t packed[16];
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    float4 sc = post4[(c0 >> 2) + e4];                // same address in every lane: broadcast
                    sc.x *= rs; sc.y *= rs; sc.z *= rs; sc.w *= rs;
                    float4 ad = bias4[(c0 >> 2) + e4];
                    if (res_row) {   // residual of these four outputs (element loads: the row may be unaligned or ragged)
                        const int cbase = n0 + c0 + 4 * e4;
                        float rr[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint16_t h = cbase + u < J.Nout ? res_row[4 * e4 + u] : (uint16_t)0;
                            rr[u] = P.is_bf16 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
                        }
                        ad.x += rr[0]; ad.y += rr[1]; ad.z += rr[2]; ad.w += rr[3];
                    }
                    float v0 = __uint_as_float(r[4 * e4 + 0]) * sc.x + ad.x, v1 = __uint_as_float(r[4 * e4 + 1]) * sc.y + ad.y;
                    float v2 = __uint_as_float(r[4 * e4 + 2]) * sc.z + ad.z, v3 = __uint_as_float(r[4 * e4 + 3]) * sc.w + ad.w;
                    if (P.out_bf16) {
                        // the reference's bound for bf16 is the largest finite bf16: the saturating conversion applies it
                        // (this arithmetic, two clamps per output at half rate, was half of a large tile's epilogue)
                        asm("cvt.rn.satfinite.bf16x2.f32 %0, %1, %2;" : "=r"(packed[2 * e4]) : "f"(v1), "f"(v0));
                        asm("cvt.rn.satfinite.bf16x2.f32 %0, %1, %2;" : "=r"(packed[2 * e4 + 1]) : "f"(v3), "f"(v2));
                    } else {
                        if (P.saturate) {
                            v0 = fminf(fmaxf(v0, -lim), lim); v1 = fminf(fmaxf(v1, -lim), lim);
                            v2 = fminf(fmaxf(v2, -lim), lim); v3 = fminf(fmaxf(v3, -lim), lim);
                        }
                        const __half2 a2 = __floats2half2_rn(v0, v1), b2 = __floats2half2_rn(v2, v3);
                        packed[2 * e4] = *reinterpret_cast<const uint32_t*>(&a2);
                        packed[2 * e4 + 1] = *reinterpret_cast<const uint32_t*>(&b2);
                    }
                }
                unsigned char* dst = static_cast<unsigned char*>(J.out) + ((size_t)row * J.ld_out + n0 + c0) * 2;
                if (n0 + c0 + 32 <= J.Nout && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4)
                        reinterpret_cast<uint4*>(dst)[v4] =
                            make_uint4(packed[4 * v4], packed[4 * v4 + 1], packed[4 * v4 + 2], packed[4 * v4 + 3]);
                } else {   // ragged edge or unaligned row: element stores, statically indexed
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (n0 + c0 + e < J.Nout)
                            reinterpret_cast<uint16_t*>(dst)[e] = (uint16_t)(packed[e >> 1] >> (16 * (e & 1)));
                }
                }
            }
        }
    }
    if (J.splits > 1 && warp >= kFirstExpandWarp) {
        // Split-K tail.  Every expand thread passes both barriers whatever happened before, so an expired wait
        // elsewhere cannot leave threads behind.  The CTA that finds the other splits' arrivals at the tile's
        // counter adds the slabs up in split order (the result does not depend on arrival order).
        volatile int* last_flag = reinterpret_cast<volatile int*>(smem + kOffMisc + 8);
        const int tu = threadIdx.x - 32 * kFirstExpandWarp;
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kExpandThreads) : "memory");
        if (tu == 0) {
            int last = 0;
            if (!*abort_flag) {
                const unsigned old = atomicAdd(J.counters + tile, 1u);
                last = old == (unsigned)(J.splits - 1);
                if (last) J.counters[tile] = 0u;   // ready for the next launch
            }
            *last_flag = last;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kExpandThreads) : "memory");
        if (*last_flag) {
            __threadfence();
            const int tp4 = P.t_pad >> 2;
            const int ncols = min(kBN, J.Nout - n0);
            const float lim = P.saturate ? (P.out_bf16 ? 3.3895313892515355e+38f : 64504.0f) : 3.4e38f;
            const float* post_s = reinterpret_cast<const float*>(smem + kOffPost);
            const float* bias_s = reinterpret_cast<const float*>(smem + kOffBias);
            // Items: (column, group of four tokens).  Two items and eight splits per round keep 16 independent
            // 16-byte loads in flight per thread; the sums are formed in split order.
            constexpr int kZ = 8;
            const int nitems = ncols * tp4;
            for (int it0 = tu; it0 < nitems; it0 += 2 * kExpandThreads) {
                float4 acc[2];
                const float* src[2];
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int it = min(it0 + w * kExpandThreads, nitems - 1);   // clamped: a duplicate is not stored
                    const int col = it / tp4, r4 = it - col * tp4;
                    src[w] = J.slabs + ((size_t)n0 + col) * P.t_pad + 4 * r4;
                    acc[w] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                const size_t zstride = (size_t)J.Nout * P.t_pad;
                for (int z0 = 0; z0 < J.splits; z0 += kZ) {
                    float4 v[2][kZ];
#pragma unroll
                    for (int u = 0; u < kZ; ++u)
#pragma unroll
                        for (int w = 0; w < 2; ++w)
                            v[w][u] = z0 + u < J.splits
                                          ? __ldcg(reinterpret_cast<const float4*>(src[w] + (size_t)(z0 + u) * zstride))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < kZ; ++u)
#pragma unroll
                        for (int w = 0; w < 2; ++w) {
                            acc[w].x += v[w][u].x; acc[w].y += v[w][u].y; acc[w].z += v[w][u].z; acc[w].w += v[w][u].w;
                        }
                }
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int it = it0 + w * kExpandThreads;
                    if (it >= nitems) continue;
                    const int col = it / tp4, r4 = it - col * tp4;
                    const float sc = post_s[col], bv = bias_s[col];
                    const float o[4] = {acc[w].x, acc[w].y, acc[w].z, acc[w].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int row = 4 * r4 + j;
                        if (row < P.T) {
                            float ex = bv;
                            if (J.resid) {
                                const size_t ra = (size_t)row * J.ld_res + n0 + col;
                                ex += P.is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(J.resid)[ra])
                                                : __half2float(static_cast<const __half*>(J.resid)[ra]);
                            }
                            const float rs = J.row_exp ? exp2f((float)(P.exp_sign * J.row_exp[row])) : 1.f;
                            const float v1 = fminf(fmaxf(o[j] * (sc * rs) + ex, -lim), lim);
                            const size_t at = (size_t)row * J.ld_out + n0 + col;
                            if (P.out_bf16) static_cast<__nv_bfloat16*>(J.out)[at] = __float2bfloat16(v1);
                            else static_cast<__half*>(J.out)[at] = __float2half(v1);
                        }
                    }
                }
            }
        }
    }
    // On an expired wait, give this CTA's bulk copies in flight a bounded time to land before
    // shared memory is released.
    if (*abort_flag && threadIdx.x == 0) {
        for (unsigned i = 0; i < (1u << 20); ++i) __nanosleep(64);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------
// Per-token exponents of a bf16 linear's intermediate.  |t[tok, r]| <= max|s_mid| * sum_k |s_in[k] * x[tok, k]| =: B,
// so t * 2^e with B * 2^e <= 2^14 fits fp16 for every r, whatever the signs in V are; typical elements sit
// sqrt(K) below the bound, far above fp16's subnormal range.  One CTA per eight tokens, up to four linears (grid.y).
// ---------------------------------------------------------------------------
struct BoundJob {
    const uint16_t* x;      // [T, ldx] bf16
    long long ldx;
    const uint16_t* s_in;   // [K] bf16
    const uint16_t* s_mid;  // [R] bf16 or nullptr (ones)
    int* row_exp;           // [T]
    int K, R;
};
struct BoundParams {
    BoundJob job[kMaxGemmJobs];
    int T;
};

__global__ void __launch_bounds__(256) row_bound_kernel(const __grid_constant__ BoundParams P) {
    const BoundJob& J = P.job[blockIdx.y];
    __shared__ float s_red[8][9];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    auto bf = [](uint16_t h) { return __uint_as_float((uint32_t)h << 16); };
    // the layer's constants first (they do not depend on the previous kernel)
    float m = J.s_mid ? 0.f : 1.f;
    if (J.s_mid)
        for (int r = threadIdx.x; r < J.R; r += 256) m = fmaxf(m, fabsf(bf(J.s_mid[r])));
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations come from the previous kernel
    // every thread takes 8-column pieces of all eight tokens of the CTA: the loads of a round are independent,
    // so a row costs one memory round trip, not one per piece
    const int tok0 = blockIdx.x * 8;
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const bool vec = (reinterpret_cast<uintptr_t>(J.x) & 15u) == 0 && (J.ldx % 8) == 0 &&
                     (reinterpret_cast<uintptr_t>(J.s_in) & 15u) == 0;
    const int kvec = vec ? (J.K & ~7) : 0;
    for (int k = threadIdx.x * 8; k < kvec; k += 2048) {
        const uint4 b = *reinterpret_cast<const uint4*>(J.s_in + k);
        uint4 a[8];
#pragma unroll
        for (int t = 0; t < 8; ++t)
            a[t] = tok0 + t < P.T ? *reinterpret_cast<const uint4*>(J.x + (size_t)(tok0 + t) * J.ldx + k) : make_uint4(0, 0, 0, 0);
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const uint32_t aw[4] = {a[t].x, a[t].y, a[t].z, a[t].w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                sum[t] += fabsf(__uint_as_float(aw[i] << 16) * __uint_as_float(bw[i] << 16)) +
                          fabsf(__uint_as_float(aw[i] & 0xFFFF0000u) * __uint_as_float(bw[i] & 0xFFFF0000u));
        }
    }
    for (int k = kvec + threadIdx.x; k < J.K; k += 256) {
        const float sk = bf(J.s_in[k]);
#pragma unroll
        for (int t = 0; t < 8; ++t)
            if (tok0 + t < P.T) sum[t] += fabsf(bf(J.x[(size_t)(tok0 + t) * J.ldx + k]) * sk);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t)
        for (int o = 16; o; o >>= 1) sum[t] += __shfl_xor_sync(0xffffffffu, sum[t], o);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < 8; ++t) s_red[warp][t] = sum[t];
        s_red[warp][8] = m;
    }
    __syncthreads();
    if (threadIdx.x < 8 && tok0 + (int)threadIdx.x < P.T) {
        float total = 0.f, mm = 0.f;
        for (int w = 0; w < 8; ++w) { total += s_red[w][threadIdx.x]; mm = fmaxf(mm, s_red[w][8]); }
        const float bound = total * mm * 1.0001f;   // (rounding of the sum itself)
        int e = 0;
        if (bound > 0.f && bound < 3.0e38f) {
            int q;
            (void)frexpf(bound, &q);                // bound = f * 2^q, 0.5 <= f < 1
            e = 14 - q;
            e = e > 100 ? 100 : (e < -100 ? -100 : e);
        }
        J.row_exp[tok0 + threadIdx.x] = e;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: no link against libcuda.
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// One linear's stage as the host sees it.
struct StageJob {
    const void* a;          // activations [T, K], row stride lda elements
    long long lda;
    const void* tiles;
    const void* pre;
    const void* post;
    void* out;
    long long ld_out;
    int K, Nout;
    const void* bias;       // [Nout] or nullptr
    const void* resid;      // [T, ld_res] or nullptr
    long long ld_res;
    const int* row_exp;     // [T] per-token exponents of the intermediate or nullptr
};
// Types of a stage: scales / bias / residual, MMA operands, output; sign of the row exponents (0: none).
struct StageTypes {
    int io_bf16, a_bf16, out_bf16, exp_sign;
};

// Tile shape of a launch and the k split of each of its jobs.
struct GroupPlan {
    int mh, nh;                       // tile: 128*mh tokens x 128*nh weight rows
    int t_pad;                        // slab row length (tokens, multiple of 4)
    int tiles_total;                  // grid.x
    int max_splits;                   // grid.z
    int csplit;                       // CTAs per cluster along grid.z that share an output tile (1: no cluster)
    int tile0[kMaxGemmJobs];          // first grid.x index of each job
    int splits[kMaxGemmJobs];         // CTAs per output tile along K (1 = no split)
    int chunks_per[kMaxGemmJobs];     // 256-column chunks per split
    int counter0[kMaxGemmJobs];       // first tile counter of the job (index into the counter words)
    size_t slab0[kMaxGemmJobs];       // first slab float of the job
    size_t slab_floats;               // slab floats of the launch
};
constexpr size_t kMaxSlabBytes = (size_t)16 << 20;
// The tile counters live in words 8..63 of the 256-byte scratch header, which no other kernel writes
// (the decode kernel that may share the scratch uses words 0..2 and the bytes behind the header).
constexpr int kCounterWord0 = 8, kMaxSplitTiles = 56;
// Up to 24 tokens the k split goes over independent CTAs with slabs in global memory (any number of splits, as
// many as there are idle SMs); beyond, the serial slab reduction of the last CTA costs more than the split saves
// and the split goes over the CTAs of a cluster instead.  Qwen3-8B decode step, slabs against clusters: 16 tokens
// 3.59 against 3.76 ms, 32 tokens 3.79 against 3.73 ms, 48 tokens 4.38 against 3.83 ms.
constexpr int kMaxSplitTokens = 24;

// The four tile configurations as the host sees them.
struct KernelInfo {
    const void* fn;
    size_t smem;
    int threads;
    int pipe_bytes;   // pipeline buffers (activation + weight stages): receive space of a cluster split
    int blocks;       // 128-token x 32-column accumulator blocks of a tile
};
template <int MH, int NH>
static KernelInfo kernel_info_of() {
    using C = GemmCfg<MH, NH>;
    return {(const void*)gemm_stage_kernel<MH, NH>, (size_t)C::kSmemBytes, C::kThreads, C::kStages * (C::kABytes + C::kWBytes),
            MH * (C::kBN / 32)};
}
static KernelInfo kernel_info(int mh, int nh) {
    if (mh == 1 && nh == 1) return kernel_info_of<1, 1>();
    if (mh == 1) return kernel_info_of<1, 2>();
    if (nh == 1) return kernel_info_of<2, 1>();
    return kernel_info_of<2, 2>();
}

static int set_kernel_attributes() {
    static bool attr_set[64];
    int dev = 0;
    NQ_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        for (int mh = 1; mh <= 2; ++mh)
            for (int nh = 1; nh <= 2; ++nh) {
                const KernelInfo ki = kernel_info(mh, nh);
                NQ_CUDA_TRY(cudaFuncSetAttribute(ki.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ki.smem));
            }
        attr_set[dev & 63] = true;
    }
    return NQ_OK;
}

// CTAs of configuration (mh, nh) that can be resident at once when they are launched as clusters of `s`
// (clusters are placed inside one GPC, so this is less than the SM count for most sizes).
static int cluster_capacity(int mh, int nh, int s) {
    static int cached[2][2][9];
    int& c = cached[mh - 1][nh - 1][s];
    if (c == 0) {
        const KernelInfo ki = kernel_info(mh, nh);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, s);
        cfg.blockDim = dim3(ki.threads);
        cfg.dynamicSmemBytes = ki.smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 1; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = (unsigned)s;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (set_kernel_attributes() != NQ_OK || cudaOccupancyMaxActiveClusters(&clusters, ki.fn, &cfg) != cudaSuccess ||
            clusters <= 0) {
            (void)cudaGetLastError();
            clusters = 0;   // this cluster size cannot be launched here: the planner leaves it out
        }
        c = clusters > 0 ? clusters * s : -1;
    }
    return c > 0 ? c : 0;
}

// Tile shape (128*mh tokens x 128*nh weight rows) by a small cost model: a CTA needs a measured number of
// cycles per 64-column step (bounded by the tensor pipe for the 256 x 256 tile, by shared-memory traffic and the
// per-step waits of the issuing threads for the smaller ones); the grid runs in ceil(CTAs/resident CTAs) waves, each
// with a fixed prologue/epilogue cost.  Launches that would leave SMs idle split the k dimension of every job
// (whole 256-column chunks per CTA): above 24 tokens over the CTAs of a cluster, which add their partial sums
// through distributed shared memory; up to 24 tokens over independent CTAs with fp32 slabs in global memory, as
// far as counters and slab budget allow.
static GroupPlan plan_group(int T, int n, const int* K, const int* Nout, bool allow_split, bool allow_cluster) {
    GroupPlan pl;
    memset(&pl, 0, sizeof(pl));
    pl.mh = 1; pl.nh = 1; pl.csplit = 1;
    static const int cand[4][2] = {{1, 1}, {2, 1}, {1, 2}, {2, 2}};
    const long long sms = sm_count();
    int min_chunks = 1 << 30, max_chunks = 0;
    for (int j = 0; j < n; ++j) {
        const int c = (K[j] + 255) / 256;
        min_chunks = c < min_chunks ? c : min_chunks;
        max_chunks = c > max_chunks ? c : max_chunks;
    }
    const bool cluster_ok = allow_cluster && T > kMaxSplitTokens;
    long long best = -1;
    for (const auto& c : cand) {
        if (c[0] == 2 && T <= kBM) continue;
        long long tiles = 0;
        for (int j = 0; j < n; ++j)
            tiles += (long long)((T + kBM * c[0] - 1) / (kBM * c[0])) * ((Nout[j] + 128 * c[1] - 1) / (128 * c[1]));
        // measured cycles of the MMA thread per 64-column step (wait + issue, tensor pipe busy)
        const long long per_step = c[0] * c[1] == 4 ? 990 : (c[0] == 2 ? 580 : (c[1] == 2 ? 830 : 485));
        const long long fixed = 6000 + 2000LL * c[0] * c[1];
        const KernelInfo ki = kernel_info(c[0], c[1]);
        for (int s = 1; s <= (cluster_ok && c[0] * c[1] < 4 ? 8 : 1); ++s) {
            if (s > 1) {
                if (s > min_chunks) break;
                if ((long long)s * ((ki.blocks + s - 1) / s) * (128 * 32 * 4) > ki.pipe_bytes) continue;
            }
            const long long resident = s == 1 ? sms : cluster_capacity(c[0], c[1], s);
            if (resident <= 0) continue;
            const long long waves = (tiles * s + resident - 1) / resident;
            const long long steps = 4LL * ((max_chunks + s - 1) / s);
            const long long cost = waves * (steps * per_step + fixed + (s > 1 ? 2500 + 300LL * s : 0));
            if (best < 0 || cost < best) { best = cost; pl.mh = c[0]; pl.nh = c[1]; pl.csplit = s; }
        }
    }
    pl.t_pad = (T + 3) / 4 * 4;
    pl.max_splits = 1;
    int tiles_n[kMaxGemmJobs];
    for (int j = 0; j < n; ++j) {
        tiles_n[j] = (Nout[j] + 128 * pl.nh - 1) / (128 * pl.nh);
        pl.tile0[j] = pl.tiles_total;
        pl.tiles_total += tiles_n[j];
        pl.splits[j] = 1;
        pl.chunks_per[j] = (K[j] + 255) / 256;
    }
    if (pl.csplit > 1) {
        pl.max_splits = pl.csplit;
        for (int j = 0; j < n; ++j) pl.chunks_per[j] = ((K[j] + 255) / 256 + pl.csplit - 1) / pl.csplit;
    }
    if (allow_split && T <= kMaxSplitTokens) {
        long long want_all = sms / pl.tiles_total;   // CTAs per tile that the idle SMs allow
        int counters_used = 0;
        size_t slab_budget = kMaxSlabBytes / sizeof(float);
        for (int j = 0; j < n && want_all >= 2; ++j) {
            const int chunks = (K[j] + 255) / 256;
            const size_t per_split = (size_t)pl.t_pad * (size_t)Nout[j];
            long long want = want_all;
            const long long by_mem = (long long)((slab_budget - pl.slab_floats) / per_split);
            want = want < by_mem ? want : by_mem;
            want = want < chunks ? want : chunks;
            if (want < 2 || counters_used + tiles_n[j] > kMaxSplitTiles) continue;
            pl.chunks_per[j] = (int)((chunks + want - 1) / want);
            pl.splits[j] = (chunks + pl.chunks_per[j] - 1) / pl.chunks_per[j];
            pl.counter0[j] = counters_used;
            counters_used += tiles_n[j];
            pl.slab0[j] = pl.slab_floats;
            pl.slab_floats += (size_t)pl.splits[j] * per_split;
            pl.max_splits = pl.max_splits > pl.splits[j] ? pl.max_splits : pl.splits[j];
        }
    }
    return pl;
}

// One stage of up to four linears: out_j[T, Nout_j] = (a_j[T, K_j] . W_j^T) * post_j.  `counters` (zero
// between launches) and `slabs` may be nullptr: no k split.
static int launch_stage(const StageJob* jobs, int n, int T, StageTypes ty, int saturate, unsigned* status,
                        unsigned* counters, float* slabs, cudaStream_t stream) {
    if (n < 1 || n > kMaxGemmJobs) return NQ_ERR_UNSUPPORTED;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return NQ_ERR_UNSUPPORTED;
    int Ks[kMaxGemmJobs], Ns[kMaxGemmJobs];
    for (int j = 0; j < n; ++j) {
        const StageJob& S = jobs[j];
        if (!aligned16(S.a) || (S.lda % 8) != 0 || (S.K % 8) != 0) return NQ_ERR_ALIGN;   // TMA: 16-byte base and stride
        if (S.pre && !aligned16(S.pre)) return NQ_ERR_ALIGN;
        Ks[j] = S.K; Ns[j] = S.Nout;
    }
    { const int st_attr = set_kernel_attributes(); if (st_attr != NQ_OK) return st_attr; }
    const GroupPlan pl = plan_group(T, n, Ks, Ns, counters != nullptr && slabs != nullptr, true);
    const int mh = pl.mh, nh = pl.nh;
    const int m_tiles = (T + kBM * mh - 1) / (kBM * mh);
    GemmParams P;
    memset(&P, 0, sizeof(P));
    P.njobs = n;
    P.status = status;
    P.T = T;
    P.t_pad = pl.t_pad;
    P.is_bf16 = ty.io_bf16;
    P.a_bf16 = ty.a_bf16;
    P.out_bf16 = ty.out_bf16;
    P.exp_sign = ty.exp_sign;
    P.saturate = saturate;
    P.csplit = pl.csplit;
    for (int j = 0; j < n; ++j) {
        const StageJob& S = jobs[j];
        GemmJob& J = P.job[j];
        const cuuint64_t dims[2] = {(cuuint64_t)S.K, (cuuint64_t)T};
        const cuuint64_t strides[1] = {(cuuint64_t)S.lda * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)(kBM * mh)};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = enc(&J.map_a, ty.a_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                               2, const_cast<void*>(S.a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return NQ_ERR_UNSUPPORTED;
        J.tiles = static_cast<const uint4*>(S.tiles);
        J.pre = S.pre;
        J.post = S.post;
        J.out = S.out;
        J.ld_out = S.ld_out;
        J.row_exp = ty.exp_sign ? S.row_exp : nullptr;
        J.bias = S.bias;
        J.resid = S.resid;
        J.ld_res = S.ld_res;
        J.K = S.K; J.Nout = S.Nout;
        J.chunks = (S.K + 255) / 256;
        J.row_groups = (S.Nout + 15) / 16;
        J.splits = pl.splits[j];
        J.chunks_per = pl.chunks_per[j];
        J.tile0 = pl.tile0[j];
        J.counters = counters ? counters + pl.counter0[j] : nullptr;
        J.slabs = slabs ? slabs + pl.slab0[j] : nullptr;
    }
    const KernelInfo ki = kernel_info(mh, nh);
    const void* fn = ki.fn;
    const size_t smem_bytes = ki.smem;
    const int threads = ki.threads;
    // Programmatic stream serialization lets this grid start while the previous kernel of the stream drains
    // (see the kernel's griddepcontrol instructions).  If the driver refuses the attribute once, plain
    // launches are used from then on.
    static bool pdl_ok = true;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.tiles_total, m_tiles, pl.max_splits);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (pl.csplit > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = (unsigned)pl.csplit;
        ++na;
    }
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = pdl_ok ? na + 1 : na;
    void* args[] = {&P};
    cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
    if (e != cudaSuccess && pdl_ok) {
        (void)cudaGetLastError();
        pdl_ok = false;
        cfg.numAttrs = na;
        e = cudaLaunchKernelExC(&cfg, fn, args);
    }
    NQ_CUDA_TRY(e);
    return NQ_OK;
}

static int g_precise_intermediate = 0;   // see nq_gemm_set_precise_intermediate

}  // namespace nq

using namespace nq;

extern "C" {

// Scratch of a GEMM group: header (status word, tile counters), the intermediates t_j[T, R_j] (16-bit,
// 256-byte aligned each), the per-token exponents of each intermediate (T words each; used by bf16 linears),
// split-K slabs (shared by the two stages).
static size_t gemm_group_layout(const nq_linear_desc* d, int n, int T, size_t* t_off, size_t* slab_off,
                                size_t* exp_off = nullptr) {
    size_t off = 256;
    int K1[kMaxGemmJobs], N1[kMaxGemmJobs], K2[kMaxGemmJobs], N2[kMaxGemmJobs];
    for (int j = 0; j < n; ++j) {
        if (t_off) t_off[j] = off;
        off += ((size_t)T * (size_t)d[j].R * 2 + 255) / 256 * 256;
        K1[j] = d[j].N; N1[j] = d[j].R; K2[j] = d[j].R; N2[j] = d[j].M;
    }
    for (int j = 0; j < n; ++j) {
        if (exp_off) exp_off[j] = off;
        off += ((size_t)T * sizeof(int) + 255) / 256 * 256;
    }
    if (slab_off) *slab_off = off;
    const size_t a = plan_group(T, n, K1, N1, true, false).slab_floats, b = plan_group(T, n, K2, N2, true, false).slab_floats;
    return off + (a > b ? a : b) * sizeof(float);
}

size_t nq_gemm_group_scratch_bytes(const nq_linear_desc* d, int n_linears, int T) {
    if (!d || n_linears <= 0 || n_linears > kMaxGemmJobs || T <= 0) return 0;
    for (int j = 0; j < n_linears; ++j)
        if (d[j].N <= 0 || d[j].R <= 0 || d[j].M <= 0) return 0;
    return gemm_group_layout(d, n_linears, T, nullptr, nullptr);
}

size_t nq_gemm_scratch_bytes(int T, int N, int R, int M) {
    if (T <= 0 || N <= 0 || R <= 0 || M <= 0) return 0;
    nq_linear_desc d;
    memset(&d, 0, sizeof(d));
    d.N = N; d.R = R; d.M = M;
    return gemm_group_layout(&d, 1, T, nullptr, nullptr);
}

int nq_onebit_gemm_fwd(const void* x, const void* tiles, const void* s_in, const void* s_out, void* y,
                       void* status_word, int T, int K, int Nout, int dtype, nq_stream_t stream) {
    if (!x || !tiles || !y || !status_word) return NQ_ERR_NULL;
    if (T <= 0 || K <= 0 || Nout <= 0) return NQ_ERR_SHAPE;
    if (dtype != NQ_F16 && dtype != NQ_BF16) return NQ_ERR_DTYPE;
    if (!aligned16(tiles)) return NQ_ERR_ALIGN;
    const StageJob job = {x, K, tiles, s_in, s_out, y, Nout, K, Nout, nullptr, nullptr, 0, nullptr};
    const int b16 = dtype == NQ_BF16;
    return launch_stage(&job, 1, T, StageTypes{b16, b16, b16, 0}, 1, static_cast<unsigned*>(status_word) + 2, nullptr, nullptr,
                        as_stream(stream));
}

int nq_gemm_group_fwd(const nq_linear_desc* d, int n_linears, int T, int dtype, void* scratch,
                      size_t scratch_bytes, nq_stream_t stream) {
    if (!d || !scratch) return NQ_ERR_NULL;
    if (n_linears <= 0 || n_linears > kMaxGemmJobs) return NQ_ERR_UNSUPPORTED;
    if (T <= 0) return NQ_ERR_SHAPE;
    if (dtype != NQ_F16 && dtype != NQ_BF16) return NQ_ERR_DTYPE;
    if (!aligned16(scratch)) return NQ_ERR_ALIGN;
    for (int j = 0; j < n_linears; ++j) {
        const nq_linear_desc& L = d[j];
        if (!L.x || !L.s_in || !L.v_tiles || !L.u_tiles || !L.s_out || !L.y) return NQ_ERR_NULL;
        if (L.N <= 0 || L.R <= 0 || L.M <= 0 || L.ldx < L.N || L.ldy < L.M) return NQ_ERR_SHAPE;
        if (L.residual && L.ldr < L.M) return NQ_ERR_SHAPE;
        if (L.N % 8 || L.R % 8) return NQ_ERR_SHAPE;
        if (!aligned16(L.v_tiles) || !aligned16(L.u_tiles)) return NQ_ERR_ALIGN;
    }
    size_t t_off[kMaxGemmJobs], exp_off[kMaxGemmJobs], slab_off = 0;
    if (scratch_bytes < gemm_group_layout(d, n_linears, T, t_off, &slab_off, exp_off)) return NQ_ERR_SCRATCH;
    unsigned* status = static_cast<unsigned*>(scratch) + 2;   // same word as the GEMV header's status
    // Both stages use the same counters and slab space: a stage touches them only after the kernel before it
    // has completed (its stores come behind the dependency wait).
    unsigned* counters = static_cast<unsigned*>(scratch) + kCounterWord0;
    float* slabs = reinterpret_cast<float*>(static_cast<char*>(scratch) + slab_off);
    StageJob s1[kMaxGemmJobs], s2[kMaxGemmJobs];
    for (int j = 0; j < n_linears; ++j) {
        const nq_linear_desc& L = d[j];
        void* t = static_cast<char*>(scratch) + t_off[j];
        int* row_exp = reinterpret_cast<int*>(static_cast<char*>(scratch) + exp_off[j]);
        s1[j] = {L.x, L.ldx, L.v_tiles, L.s_in, L.s_mid, t, L.R, L.N, L.R, nullptr, nullptr, 0, row_exp};
        s2[j] = {t, L.R, L.u_tiles, nullptr, L.s_out, L.y, L.ldy, L.R, L.M, L.bias, L.residual, L.ldr, row_exp};
    }
    if (dtype == NQ_F16 || !g_precise_intermediate) {   // the intermediate in the I/O type, as it comes
        const int b16 = dtype == NQ_BF16;
        const StageTypes ty = {b16, b16, b16, 0};
        const int st = launch_stage(s1, n_linears, T, ty, 0, status, counters, slabs, as_stream(stream));
        if (st != NQ_OK) return st;
        return launch_stage(s2, n_linears, T, ty, 1, status, counters, slabs, as_stream(stream));
    }
    // bf16 with the precise intermediate switched on: a bf16 intermediate carries 8 significant bits into stage 2
    // (its rounding alone is up to 1.6e-3 of the output's maximum); here it is kept as fp16 times a per-token
    // power of two instead.  row_bound_kernel finds the exponents from a bound on |t| that holds for any signs;
    // stage 2 then runs as an fp16 MMA on +-1 weights.  One more small kernel per launch group.
    {
        BoundParams B;
        memset(&B, 0, sizeof(B));
        B.T = T;
        for (int j = 0; j < n_linears; ++j) {
            const nq_linear_desc& L = d[j];
            B.job[j] = {static_cast<const uint16_t*>(L.x), L.ldx, static_cast<const uint16_t*>(L.s_in),
                        static_cast<const uint16_t*>(L.s_mid), const_cast<int*>(s1[j].row_exp), L.N, L.R};
        }
        static bool pdl_ok = true;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((T + 7) / 8), (unsigned)n_linears);
        cfg.blockDim = dim3(256);
        cfg.stream = as_stream(stream);
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = pdl_ok ? 1 : 0;
        void* args[] = {&B};
        cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)row_bound_kernel, args);
        if (e != cudaSuccess && pdl_ok) {
            (void)cudaGetLastError();
            pdl_ok = false;
            cfg.numAttrs = 0;
            e = cudaLaunchKernelExC(&cfg, (const void*)row_bound_kernel, args);
        }
        NQ_CUDA_TRY(e);
    }
    const int st = launch_stage(s1, n_linears, T, StageTypes{1, 1, 0, +1}, 0, status, counters, slabs, as_stream(stream));
    if (st != NQ_OK) return st;
    return launch_stage(s2, n_linears, T, StageTypes{1, 0, 1, -1}, 1, status, counters, slabs, as_stream(stream));
}

int nq_gemm_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid, const void* u_tiles,
                const void* s_out, void* y, void* scratch, size_t scratch_bytes, int T, int N, int R, int M,
                int dtype, nq_stream_t stream) {
    if (!x || !s_in || !v_tiles || !u_tiles || !s_out || !y || !scratch) return NQ_ERR_NULL;
    if (T <= 0 || N <= 0 || R <= 0 || M <= 0) return NQ_ERR_SHAPE;
    nq_linear_desc d;
    memset(&d, 0, sizeof(d));
    d.x = x; d.s_in = s_in; d.v_tiles = v_tiles; d.s_mid = s_mid; d.u_tiles = u_tiles; d.s_out = s_out;
    d.y = y; d.N = N; d.R = R; d.M = M; d.ldx = N; d.ldy = M;
    return nq_gemm_group_fwd(&d, 1, T, dtype, scratch, scratch_bytes, stream);
}


int nq_gemm_set_precise_intermediate(int on) {
    const int old = g_precise_intermediate;
    g_precise_intermediate = on ? 1 : 0;
    return old;
}

// One decode launch handles four tokens; from five tokens on the split-K GEMM is faster than two launches.
int nq_gemv_max_tokens(void) { return 4; }

size_t nq_linear_scratch_bytes(int T, int N, int R, int M) {
    const size_t a = nq_gemv_scratch_bytes(T, N, R, M), b = nq_gemm_scratch_bytes(T, N, R, M);
    return a > b ? a : b;
}

int nq_linear_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid, const void* u_tiles,
                  const void* s_out, void* y, void* scratch, size_t scratch_bytes, int T, int N, int R, int M,
                  int dtype, nq_stream_t stream) {
    if (T <= nq_gemv_max_tokens() || (N % 8) || (R % 8))
        return nq_gemv_fwd(x, s_in, v_tiles, s_mid, u_tiles, s_out, y, scratch, scratch_bytes, T, N, R, M, dtype,
                           stream);
    return nq_gemm_fwd(x, s_in, v_tiles, s_mid, u_tiles, s_out, y, scratch, scratch_bytes, T, N, R, M, dtype, stream);
}

}  // extern "C"
