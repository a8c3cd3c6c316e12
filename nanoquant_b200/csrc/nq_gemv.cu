// Decode GEMV for the binary low-rank linear, one launch per group of linears.
//
//   y = s_out * (U . (s_mid * (V . (s_in * x))))          T <= 4 tokens per launch
//
// The kernel is bound by the HBM stream of the packed factors; everything else is
// arranged so that the per-weight instruction cost stays far below that stream:
//
//  * The input vector of a phase (s_in*x, or the rank-R intermediate t) is turned,
//    once per CTA, into 16-bit fixed point with a per-token scale and split into
//    two int8 terms (hi, lo).  These 2*T int8 vectors are the B operand (the N=8
//    columns) of an integer tensor-core MMA (mma.sync m16n8k32 s8*s8->s32).
//  * The packed sign bits are the A operand WITHOUT unpacking: in the tile layout
//    (see nq_rows_to_tiles) `word & (0x01010101 << j)` is an int8x4 register with
//    values {0, 2^j}, so one LOP3 prepares four weights and eight masks j = 0..7
//    consume a whole 32-bit word.  Each mask has its own accumulator; the sums are
//    recombined exactly with shifts at the end of a row tile.
//  * sum(+-X) = sum(X) - 2 * sum_{bit=1}(X); all accumulation is exact int32, so the
//    result does not depend on the order in which warps add their parts.
//
// A legacy SIMT sign-flip-add inner loop issues ~1.5 instructions per weight and
// tops out near one third of the HBM rate on this part, which is why the integer
// MMA is used as a wide dot-product unit here.  No floating-point tensor math and
// no shared-memory staging of the weights is involved: each lane streams its tile
// words with 128-bit loads straight into the registers that feed the MMA.
//
// Phases: phase 1 computes t[T,R] (fp32, in scratch), a device-wide barrier
// follows, phase 2 computes y.  Several linears that share the two phases (q/k/v,
// gate/up) are processed in one launch.  The barrier spin is bounded: on expiry a
// status word is set and every CTA returns.
//
// replaces: src/nanoquant/kernel/cuda/gemv_kernel.cu:43-301 of the reference
// (two kernels per linear, fp16/bf16 accumulation, sign-flip adds).
#include "nq_common.cuh"

namespace nq {

#ifndef NQ_GEMV_THREADS
#define NQ_GEMV_THREADS 512
#endif
#ifndef NQ_GEMV_STAGES
#define NQ_GEMV_STAGES 4
#endif
constexpr int kGemvThreads = NQ_GEMV_THREADS;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxJobs = 4;         // linears per launch
constexpr int kMaxTok = 4;          // tokens per launch (2 int8 terms each -> 8 MMA columns)
constexpr int kQMax = 32639;        // 127*256 + 127: hi and lo both fit a signed byte
constexpr int kStages = NQ_GEMV_STAGES;          // 1 KB weight slots in flight per warp
constexpr size_t kRedBytes = 384;   // per-warp maxima (kGemvWarps * 4 floats) + 4 inverse scales
constexpr size_t kFixedBytes = 512;
constexpr size_t kRingBytes = (size_t)kGemvWarps * kStages * 1024;
constexpr unsigned kSpinLimit = 4000000u;
constexpr size_t kHeaderBytes = 256;

enum : int { KIND_F16 = 0, KIND_BF16 = 1, KIND_F32 = 2 };

#ifdef NQ_GEMV_TRACE  // development aid: per-CTA (id, timestamp) records of the phase steps
__device__ unsigned long long g_trace[148 * 64];
__device__ int g_trace_n[148];
__device__ __forceinline__ void trace_mark(int id) {
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const int n = g_trace_n[blockIdx.x];
        if (n < 64) { g_trace[blockIdx.x * 64 + n] = (t << 8) | (unsigned)id; g_trace_n[blockIdx.x] = n + 1; }
    }
}
#define NQ_TRACE(id) trace_mark(id)
#else
#define NQ_TRACE(id) ((void)0)
#endif

struct Job {
    const uint4* tiles;   // [row_groups][chunks][32]
    const void* in;       // [T, ld_in]  fp16/bf16 (phase 1) or fp32 (phase 2)
    const void* pre;      // [K] scale in the I/O dtype, or nullptr
    const void* post;     // [rows] scale in the I/O dtype, or nullptr
    void* out;            // [T, ld_out] fp32 (phase 1) or fp16/bf16 (phase 2)
    long long ld_in, ld_out;
    int rows, K;
    int chunks;           // ceil(K / 256)
    int items;            // ceil(rows / 32)
    int in_kind, out_kind;
    int vec;              // rows of `in` / `pre` are 16-byte aligned and K % 8 == 0
};

struct Phase {
    Job job[kMaxJobs];
    int njobs;
};

struct GemvParams {
    Phase phase[2];
    unsigned* header;     // [0] barrier count, [1] barrier generation, [2] status
    int T;
    int scale_kind;       // dtype of the scale vectors (KIND_F16 / KIND_BF16)
    int xq_stride;        // bytes between the int8 vectors in shared memory
    int max_items;        // row tiles a CTA may own per job
};

__device__ __forceinline__ float load_as_float(const void* p, long long i, int kind) {
    if (kind == KIND_F16) return __half2float(static_cast<const __half*>(p)[i]);
    if (kind == KIND_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return __ldcg(static_cast<const float*>(p) + i);  // written by other CTAs of this launch: bypass L1
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_tile(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Bounded device-wide barrier on {count, generation} words.  Returns false when the
// wait expired (a status word is set and the caller returns).  One thread per CTA
// arrives with a release and polls with acquires; the CTA barrier before and after
// extends the ordering to every thread of the CTA.
__device__ bool grid_barrier(unsigned* header, unsigned nblocks) {
    __shared__ int ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        ok = 1;
        unsigned my_gen, old;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(my_gen) : "l"(header + 1) : "memory");
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(header) : "memory");
        if (old == nblocks - 1) {
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(header), "r"(0u) : "memory");
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(header + 1) : "memory");
        } else {
            unsigned spins = 0, cur;
            while (true) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(cur) : "l"(header + 1) : "memory");
                if (cur != my_gen) break;
                if (++spins > kSpinLimit) {
                    atomicExch(header + 2, (unsigned)(-NQ_ERR_TIMEOUT));
                    ok = 0;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return ok != 0;
}

// Eight consecutive elements of a vector as floats (one or two 128-bit loads).
template <int KIND>
__device__ __forceinline__ void load8(const void* base, long long i, float (&v)[8]) {
    if (KIND == KIND_F32) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + i));
        const float4 b = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + i) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + i);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (KIND == KIND_F16) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                v[2 * e] = f.x; v[2 * e + 1] = f.y;
            } else {  // bf16 -> fp32 is a 16-bit shift
                v[2 * e] = __uint_as_float(w[e] << 16);
                v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
            }
        }
    }
}

// Quantise the input vectors of a job into shared memory.
//   xq: 2*T int8 vectors (row 2*tok = hi term, 2*tok+1 = lo term), `stride` bytes apart,
//       in the k order the MMA B fragments expect (see below); columns K..Kpad are zero.
//   sumx[tok]: sum of the 16-bit values, delta[tok]: value of one unit.
// Byte position inside a chunk of 256 columns: 32*j + 8*q + 4*h + b for column
// 32*j + 16*h + 4*q + b, so that lane (g, q) fetches its two B registers
// {k = 4q.., k = 16+4q..} of mask j with one 64-bit load.
// The code is kept as small loops on purpose: it runs once per phase, where
// instruction fetch, not arithmetic, sets the pace.
//
// Vector path: rows of `in` / `pre` 16-byte aligned, K % 8 == 0; eight columns per thread and step.
template <int IN_KIND>
__device__ __noinline__ void quantise_vec(const Job& jb, int T, int8_t* xq, int stride, float* red,
                                          int* sumx, float* delta) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, Kpad = jb.chunks * 256;
    constexpr bool kHasPre = (IN_KIND != KIND_F32);
    // pass 1: per-token max |in * pre|
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float m = 0.f;
#pragma unroll 1
        for (int k8 = tid * 8; k8 < K; k8 += kGemvThreads * 8) {
            float v[8], s[8];
            load8<IN_KIND>(jb.in, t * jb.ld_in + k8, v);
            if (kHasPre) load8<IN_KIND>(jb.pre, k8, s);
#pragma unroll
            for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(kHasPre ? v[e] * s[e] : v[e]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red[warp * kMaxTok + t] = m;
    }
    __syncthreads();
    if (tid < T) {
        float m = 0.f;
        for (int w = 0; w < kGemvWarps; ++w) m = fmaxf(m, red[w * kMaxTok + tid]);
        // a non-finite or zero maximum quantises everything to zero
        const bool good = (m > 0.f) && (m < 3.0e38f);
        red[kGemvWarps * kMaxTok + tid] = good ? (float)kQMax / m : 0.f;
        delta[tid] = good ? m / (float)kQMax : 0.f;
        sumx[tid] = 0;
    }
    __syncthreads();
    // pass 2: |p * inv| <= kQMax + 2^-8 by construction (same products as in pass 1), no clamp needed
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float inv = red[kGemvWarps * kMaxTok + t];
        int8_t* rh = xq + (2 * t) * stride;
        int8_t* rl = rh + stride;
        int acc = 0;
#pragma unroll 1
        for (int k8 = tid * 8; k8 < Kpad; k8 += kGemvThreads * 8) {
            int X[8];
            if (k8 < K) {
                float v[8], s[8];
                load8<IN_KIND>(jb.in, t * jb.ld_in + k8, v);
                if (kHasPre) load8<IN_KIND>(jb.pre, k8, s);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    X[e] = __float2int_rn((kHasPre ? v[e] * s[e] : v[e]) * inv);
                    acc += X[e];
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) X[e] = 0;
            }
            // X = 256 * hi + lo with lo the signed low byte: lo = byte 0 of X, hi = byte 1 of X + 128
            uint32_t lo[2], hi[2];
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                const uint32_t x0 = X[4 * w], x1 = X[4 * w + 1], x2 = X[4 * w + 2], x3 = X[4 * w + 3];
                lo[w] = __byte_perm(__byte_perm(x0, x1, 0x0040), __byte_perm(x2, x3, 0x0040), 0x5410);
                hi[w] = __byte_perm(__byte_perm(x0 + 128u, x1 + 128u, 0x0051),
                                    __byte_perm(x2 + 128u, x3 + 128u, 0x0051), 0x5410);
            }
            const int kin = k8 & 255;  // j = kin >> 5, h = (kin >> 4) & 1, q = (kin >> 2) & 3 (0 or 2)
            const int pos = (k8 & ~255) + (kin & 0xE0) + 2 * (kin & 8) + ((kin & 16) >> 2);
            *reinterpret_cast<uint32_t*>(rh + pos) = hi[0];
            *reinterpret_cast<uint32_t*>(rh + pos + 8) = hi[1];
            *reinterpret_cast<uint32_t*>(rl + pos) = lo[0];
            *reinterpret_cast<uint32_t*>(rl + pos + 8) = lo[1];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0 && acc != 0) atomicAdd(&sumx[t], acc);
    }
    __syncthreads();
}

// Scalar path for unaligned or ragged inputs (any K, any alignment).
__device__ __noinline__ void quantise_scalar(const Job& jb, int T, int scale_kind, int8_t* xq, int stride,
                                             float* red, int* sumx, float* delta) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, Kpad = jb.chunks * 256;
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float m = 0.f;
        for (int k = tid; k < K; k += kGemvThreads) {
            const float s = jb.pre ? load_as_float(jb.pre, k, scale_kind) : 1.f;
            m = fmaxf(m, fabsf(load_as_float(jb.in, t * jb.ld_in + k, jb.in_kind) * s));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red[warp * kMaxTok + t] = m;
    }
    __syncthreads();
    if (tid < T) {
        float m = 0.f;
        for (int w = 0; w < kGemvWarps; ++w) m = fmaxf(m, red[w * kMaxTok + tid]);
        const bool good = (m > 0.f) && (m < 3.0e38f);
        red[kGemvWarps * kMaxTok + tid] = good ? (float)kQMax / m : 0.f;
        delta[tid] = good ? m / (float)kQMax : 0.f;
        sumx[tid] = 0;
    }
    __syncthreads();
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float inv = red[kGemvWarps * kMaxTok + t];
        int acc = 0;
        for (int k = tid; k < Kpad; k += kGemvThreads) {
            int X = 0;
            if (k < K) {
                const float s = jb.pre ? load_as_float(jb.pre, k, scale_kind) : 1.f;
                X = __float2int_rn(load_as_float(jb.in, t * jb.ld_in + k, jb.in_kind) * s * inv);
            }
            acc += X;
            const int kin = k & 255;
            const int pos = (k & ~255) + (kin & 0xE0) + 2 * (kin & 12) + ((kin & 16) >> 2) + (kin & 3);
            xq[(2 * t) * stride + pos] = (int8_t)((X + 128) >> 8);
            xq[(2 * t + 1) * stride + pos] = (int8_t)(X & 0xFF);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0 && acc != 0) atomicAdd(&sumx[t], acc);
    }
    __syncthreads();
}

__device__ __forceinline__ void quantise_input(const Job& jb, int T, int scale_kind, int8_t* xq, int stride,
                                               float* red, int* sumx, float* delta) {
    if (!jb.vec) quantise_scalar(jb, T, scale_kind, xq, stride, red, sumx, delta);
    else if (jb.in_kind == KIND_F32) quantise_vec<KIND_F32>(jb, T, xq, stride, red, sumx, delta);
    else if (jb.in_kind == KIND_F16) quantise_vec<KIND_F16>(jb, T, xq, stride, red, sumx, delta);
    else quantise_vec<KIND_BF16>(jb, T, xq, stride, red, sumx, delta);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One phase: every CTA walks the jobs; inside a job it owns the row tiles (32 rows)
// blockIdx.x, blockIdx.x + gridDim.x, ... and its warps split the K chunks of those
// tiles.  Each warp streams its (tile, chunk) pairs - 1 KB of packed weights each -
// through a private ring of kStages shared-memory slots filled with cp.async, so the
// loop body exists once and stays small enough for the instruction cache.
__device__ __noinline__ void run_phase(const Phase& ph, const GemvParams& P, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    // shared memory carve-up
    float* red = reinterpret_cast<float*>(smem);                          // [warps][4]
    int* sumx = reinterpret_cast<int*>(smem + kRedBytes);                 // [4]
    float* delta = reinterpret_cast<float*>(smem + kRedBytes + 16);       // [4]
    uint4* ring = reinterpret_cast<uint4*>(smem + kFixedBytes) + warp * (kStages * 64);  // [stage][2][32]
    int* s1 = reinterpret_cast<int*>(smem + kFixedBytes + kRingBytes);    // [max_items][4][32]
    int8_t* xq = reinterpret_cast<int8_t*>(smem + kFixedBytes + kRingBytes + (size_t)P.max_items * 512);

#pragma unroll 1
    for (int ji = 0; ji < ph.njobs; ++ji) {
        const Job& jb = ph.job[ji];
        const int my_items = ((int)blockIdx.x < jb.items)
                                 ? (jb.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        if (my_items == 0) continue;  // uniform per CTA
        const int chunks = jb.chunks;
        const int row_groups = (jb.rows + 15) >> 4;
        // The CTA's (tile, chunk) pairs, tile-major, are split into one contiguous range per
        // warp: a warp then streams consecutive memory and folds its partial sums into shared
        // memory only when it leaves a row tile (at most twice more often than it has tiles).
        const int npairs = my_items * chunks;
        const int p_begin = (int)((long long)npairs * warp / kGemvWarps);
        const int p_end = (int)((long long)npairs * (warp + 1) / kGemvWarps);
        const int my_pairs = p_end - p_begin;

        // load stream state: (item, chunk) of the next pair to fetch
        int l_il = p_begin / chunks, l_c = p_begin - l_il * chunks, l_n = 0;
        auto issue_load = [&]() {
            if (l_n < my_pairs) {
                const int rg = 2 * ((int)blockIdx.x + l_il * (int)gridDim.x);
                const int rgb = (rg + 1 < row_groups) ? rg + 1 : rg;  // odd tail: re-read, result discarded
                uint4* dst = ring + (l_n % kStages) * 64 + lane;
                cp_async16(dst, jb.tiles + ((size_t)rg * chunks + l_c) * 32 + lane);
                cp_async16(dst + 32, jb.tiles + ((size_t)rgb * chunks + l_c) * 32 + lane);
                if (++l_c == chunks) { l_c = 0; ++l_il; }
                ++l_n;
            }
            cp_async_commit();  // always commit so that group counting stays uniform
        };
        // the first weight loads do not depend on the input vector: issue them before it is prepared
#pragma unroll
        for (int d = 0; d < kStages - 1; ++d) issue_load();

        NQ_TRACE(1);
        for (int i = tid; i < my_items * 128; i += kGemvThreads) s1[i] = 0;
        quantise_input(jb, P.T, P.scale_kind, xq, P.xq_stride, red, sumx, delta);
        NQ_TRACE(5);

        const int brow = (g < 2 * P.T) ? g : (2 * P.T - 1);  // unused MMA columns re-read a valid vector
        const int8_t* bbase = xq + brow * P.xq_stride + 8 * q;

        int accA[8][4], accB[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) { accA[j][i] = 0; accB[j][i] = 0; }
        int c_il = p_begin / chunks, c_c = p_begin - c_il * chunks;
#pragma unroll 1
        for (int n = 0; n < my_pairs; ++n) {
            issue_load();
            cp_async_wait<kStages - 1>();
            __syncwarp();
            const uint4* slot = ring + (n % kStages) * 64 + lane;
            const uint4 ta = slot[0], tb = slot[32];
            const uint2* bp = reinterpret_cast<const uint2*>(bbase + c_c * 256);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint2 b = bp[j * 4];
                const uint32_t m = 0x01010101u << j;
                mma_s8(accA[j], ta.x & m, ta.y & m, ta.z & m, ta.w & m, b.x, b.y);
                mma_s8(accB[j], tb.x & m, tb.y & m, tb.z & m, tb.w & m, b.x, b.y);
            }
            __syncwarp();  // every lane has read the slot before it is refilled
            // when this warp leaves the row tile, fold its partial sums into shared memory
            if (++c_c == chunks || n + 1 == my_pairs) {
                // d_j = 2^j * sum (j < 7), -128 * sum (j = 7): exact shifts
                int v[4] = {0, 0, 0, 0};  // {rows g, g+8 of group A, rows g, g+8 of group B}
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int sg = (j == 7) ? -1 : 1;
                    v[0] += sg * ((accA[j][0] >> j) * 256 + (accA[j][1] >> j));
                    v[1] += sg * ((accA[j][2] >> j) * 256 + (accA[j][3] >> j));
                    v[2] += sg * ((accB[j][0] >> j) * 256 + (accB[j][1] >> j));
                    v[3] += sg * ((accB[j][2] >> j) * 256 + (accB[j][3] >> j));
#pragma unroll
                    for (int i = 0; i < 4; ++i) { accA[j][i] = 0; accB[j][i] = 0; }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (v[i] != 0) atomicAdd(&s1[(c_il * 4 + i) * 32 + lane], v[i]);
                if (c_c == chunks) { c_c = 0; ++c_il; }
            }
        }
        cp_async_wait<0>();
        __syncthreads();
        NQ_TRACE(6);
        // finalise: thread -> (item, v, lane); lane (g, q) holds token q of rows g / g+8
        for (int i = tid; i < my_items * 128; i += kGemvThreads) {
            const int il = i >> 7, v = (i >> 5) & 3, ln = i & 31;
            const int tok = ln & 3, gg = ln >> 2;
            const int row = 32 * ((int)blockIdx.x + il * (int)gridDim.x) + 16 * (v >> 1) + 8 * (v & 1) + gg;
            if (tok < P.T && row < jb.rows) {
                const long long r = (long long)sumx[tok] - 2LL * (long long)s1[i];
                float val = (float)r * delta[tok];
                if (jb.post) val *= load_as_float(jb.post, row, P.scale_kind);
                if (jb.out_kind == KIND_F32) {
                    static_cast<float*>(jb.out)[tok * jb.ld_out + row] = val;
                } else if (jb.out_kind == KIND_F16) {
                    // same saturation bounds as the reference epilogue
                    val = fminf(fmaxf(val, -64504.0f), 64504.0f);
                    static_cast<__half*>(jb.out)[tok * jb.ld_out + row] = __float2half(val);
                } else {
                    val = fminf(fmaxf(val, -3.3895313892515355e+38f), 3.3895313892515355e+38f);
                    static_cast<__nv_bfloat16*>(jb.out)[tok * jb.ld_out + row] = __float2bfloat16(val);
                }
            }
        }
        __syncthreads();  // xq / s1 are reused by the next job
        NQ_TRACE(7);
    }
}

__global__ void __launch_bounds__(kGemvThreads, 1) gemv_group_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(16) unsigned char smem[];
    // The descriptors are read with runtime indices; one cooperative copy out of the
    // parameter bank into shared memory replaces many serial constant-cache misses.
    __shared__ __align__(16) Phase sphase[2];
#ifdef NQ_GEMV_TRACE
    if (threadIdx.x == 0) g_trace_n[blockIdx.x] = 0;
#endif
    NQ_TRACE(0);
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&P.phase[0]);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&sphase[0]);
        for (int i = threadIdx.x; i < (int)(sizeof(Phase) * 2 / 4); i += kGemvThreads) dst[i] = src[i];
        __syncthreads();
    }
#pragma unroll 1
    for (int ph = 0; ph < 2; ++ph) {
        run_phase(sphase[ph], P, smem);
        NQ_TRACE(8);
        if (ph == 0 && !grid_barrier(P.header, gridDim.x)) return;
        NQ_TRACE(9);
    }
}

static size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

}  // namespace nq

using namespace nq;

extern "C" {

size_t nq_gemv_scratch_bytes(int T, int N, int R, int M) {
    if (T <= 0 || N <= 0 || R <= 0 || M <= 0) return 0;
    return kHeaderBytes + round_up((size_t)kMaxTok * (size_t)R * sizeof(float), 256);
}

size_t nq_gemv_group_scratch_bytes(const nq_linear_desc* d, int n_linears, int T) {
    if (!d || n_linears <= 0 || n_linears > kMaxJobs || T <= 0) return 0;
    size_t b = kHeaderBytes;
    for (int i = 0; i < n_linears; ++i) {
        if (d[i].R <= 0) return 0;
        b += round_up((size_t)kMaxTok * (size_t)d[i].R * sizeof(float), 256);
    }
    return b;
}

int nq_gemv_group_fwd(const nq_linear_desc* d, int n_linears, int T, int dtype, void* scratch,
                      size_t scratch_bytes, nq_stream_t stream) {
    if (!d || !scratch) return NQ_ERR_NULL;
    if (n_linears <= 0 || n_linears > kMaxJobs) return NQ_ERR_UNSUPPORTED;
    if (T <= 0) return NQ_ERR_SHAPE;
    if (dtype != NQ_F16 && dtype != NQ_BF16) return NQ_ERR_DTYPE;
    if (!aligned16(scratch)) return NQ_ERR_ALIGN;
    if (scratch_bytes < nq_gemv_group_scratch_bytes(d, n_linears, T)) return NQ_ERR_SCRATCH;

    int maxK = 0;
    for (int i = 0; i < n_linears; ++i) {
        const nq_linear_desc& L = d[i];
        if (!L.x || !L.s_in || !L.v_tiles || !L.u_tiles || !L.s_out || !L.y) return NQ_ERR_NULL;
        if (L.N <= 0 || L.R <= 0 || L.M <= 0) return NQ_ERR_SHAPE;
        if (L.ldx < L.N || L.ldy < L.M) return NQ_ERR_SHAPE;
        if (!aligned16(L.v_tiles) || !aligned16(L.u_tiles)) return NQ_ERR_ALIGN;
        maxK = L.N > maxK ? L.N : maxK;
        maxK = L.R > maxK ? L.R : maxK;
    }
    int dev = 0;
    NQ_CUDA_TRY(cudaGetDevice(&dev));
    const int sms = sm_count();
    static int smem_optin[64];
    if (smem_optin[dev & 63] == 0) {
        int v = 0;
        NQ_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        cudaFuncAttributes fa;
        NQ_CUDA_TRY(cudaFuncGetAttributes(&fa, gemv_group_kernel));
        v -= (int)fa.sharedSizeBytes;  // the opt-in limit covers static + dynamic shared memory
        NQ_CUDA_TRY(cudaFuncSetAttribute(gemv_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
        smem_optin[dev & 63] = v;
    }
    const int grid = sms;
    int max_items = 1;
    for (int i = 0; i < n_linears; ++i) {
        const int it1 = ((d[i].R + 31) / 32 + grid - 1) / grid, it2 = ((d[i].M + 31) / 32 + grid - 1) / grid;
        max_items = it1 > max_items ? it1 : max_items;
        max_items = it2 > max_items ? it2 : max_items;
    }
    const int kpad = (maxK + 255) / 256 * 256;
    const int stride = kpad + 32;  // 32 mod 128: conflict-free 64-bit fragment loads

    // tokens are processed in groups that fit the 8 MMA columns and shared memory
    int tg = T < kMaxTok ? T : kMaxTok;
    auto smem_for = [&](int t) { return kFixedBytes + kRingBytes + (size_t)max_items * 512 + (size_t)2 * t * stride; };
    while (tg > 1 && smem_for(tg) > (size_t)smem_optin[dev & 63]) --tg;
    if (smem_for(tg) > (size_t)smem_optin[dev & 63]) return NQ_ERR_UNSUPPORTED;

    const size_t esz = 2;
    for (int t0 = 0; t0 < T; t0 += tg) {
        const int tn = (T - t0) < tg ? (T - t0) : tg;
        GemvParams P;
        memset(&P, 0, sizeof(P));
        P.header = static_cast<unsigned*>(scratch);
        P.T = tn;
        P.scale_kind = dtype;
        P.xq_stride = stride;
        P.max_items = max_items;
        P.phase[0].njobs = P.phase[1].njobs = n_linears;
        size_t off = kHeaderBytes;
        for (int i = 0; i < n_linears; ++i) {
            const nq_linear_desc& L = d[i];
            float* tbuf = reinterpret_cast<float*>(static_cast<char*>(scratch) + off);
            off += round_up((size_t)kMaxTok * (size_t)L.R * sizeof(float), 256);
            Job& a = P.phase[0].job[i];
            a.tiles = static_cast<const uint4*>(L.v_tiles);
            a.in = static_cast<const char*>(L.x) + (size_t)t0 * L.ldx * esz;
            a.pre = L.s_in;
            a.post = L.s_mid;
            a.out = tbuf;
            a.ld_in = L.ldx;
            a.ld_out = L.R;
            a.rows = L.R;
            a.K = L.N;
            a.chunks = (L.N + 255) / 256;
            a.items = (L.R + 31) / 32;
            a.in_kind = dtype;
            a.out_kind = KIND_F32;
            a.vec = (L.N % 8 == 0) && (L.ldx % 8 == 0) && aligned16(a.in) && aligned16(L.s_in);
            Job& b = P.phase[1].job[i];
            b.tiles = static_cast<const uint4*>(L.u_tiles);
            b.in = tbuf;
            b.pre = nullptr;
            b.post = L.s_out;
            b.out = static_cast<char*>(L.y) + (size_t)t0 * L.ldy * esz;
            b.ld_in = L.R;
            b.ld_out = L.ldy;
            b.rows = L.M;
            b.K = L.R;
            b.chunks = (L.R + 255) / 256;
            b.items = (L.M + 31) / 32;
            b.in_kind = KIND_F32;
            b.out_kind = dtype;
            b.vec = (L.R % 8 == 0);  // the intermediate lives in the 256-byte aligned scratch
        }
        void* args[] = {&P};
        NQ_CUDA_TRY(cudaLaunchCooperativeKernel((const void*)gemv_group_kernel, dim3(grid), dim3(kGemvThreads),
                                                args, smem_for(tn), as_stream(stream)));
    }
    return NQ_OK;
}

int nq_gemv_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                const void* u_tiles, const void* s_out, void* y, void* scratch, size_t scratch_bytes,
                int T, int N, int R, int M, int dtype, nq_stream_t stream) {
    nq_linear_desc d;
    d.x = x; d.s_in = s_in; d.v_tiles = v_tiles; d.s_mid = s_mid; d.u_tiles = u_tiles; d.s_out = s_out;
    d.y = y; d.N = N; d.R = R; d.M = M; d.ldx = N; d.ldy = M;
    return nq_gemv_group_fwd(&d, 1, T, dtype, scratch, scratch_bytes, stream);
}

#ifdef NQ_GEMV_TRACE
int nq_debug_read_trace(unsigned long long* host_out) {
    NQ_CUDA_TRY(cudaDeviceSynchronize());
    NQ_CUDA_TRY(cudaMemcpyFromSymbol(host_out, g_trace, sizeof(unsigned long long) * 148 * 64));
    return NQ_OK;
}
#endif

int nq_scratch_status(const void* scratch, nq_stream_t stream) {
    if (!scratch) return NQ_ERR_NULL;
    unsigned h[4] = {0, 0, 0, 0};
    NQ_CUDA_TRY(cudaMemcpyAsync(h, scratch, sizeof(h), cudaMemcpyDeviceToHost, as_stream(stream)));
    NQ_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    return h[2] == 0 ? NQ_OK : -(int)h[2];
}

}  // extern "C"
