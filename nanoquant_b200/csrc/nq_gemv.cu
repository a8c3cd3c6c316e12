// Decode GEMV for the binary low-rank linear, one launch per group of linears.
//
//   y = s_out * (U . (s_mid * (V . (s_in * x)))) (+ bias) (+ residual)        T <= 4 tokens per launch
//
// The kernel is bound by the HBM stream of the packed factors and, for the layer sizes of 8B-class
// decoders, by a chain of dependent latencies (memory round trips of 0.4-0.9 us each, CTA barriers).
//
//  * The packed sign bits are the A operand of an integer tensor-core MMA (mma.sync m16n8k32
//    s8*s8->s32) WITHOUT unpacking: in the tile layout (see nq_rows_to_tiles)
//    `word & (0x01010101 << j)` is an int8x4 register with values {0, 2^j} ({0, -128} for j = 7), so
//    one LOP3 prepares four weights and the eight masks j = 0..7 consume a whole 32-bit word.  Columns
//    [32j, 32j+32) of a 256-column chunk form the "class" j.
//  * The input vector of a phase (s_in*x, or the rank-R intermediate t) is turned, once per CTA, into
//    17-bit fixed point X with a per-token scale.  A column of class j is stored as X * 2^(7-j)
//    (negated for j = 7), split into three signed bytes.  The product of the A value 2^j and that
//    operand is 2^7 * X for every class, so all eight masks accumulate into ONE accumulator per output
//    row and byte term.  The three byte terms of a token are three of the N = 8 MMA columns.
//  * sum(+-X) = sum(X) - 2 * sum_{bit=1}(X).  All accumulation is exact int32 / int64, so a result does
//    not depend on how rows are dealt to warps, CTAs or launches.
//
// A SIMT sign-flip-add inner loop issues ~1.5 instructions per weight and tops out near one third of
// the HBM rate on this part, which is why the integer MMA is used as a wide dot-product unit here.
//
// Launch structure.  Phase 1 computes t[T,R] (fp32), phase 2 computes y; the linears of a group (q/k/v,
// gate/up) go through both phases together.  In each phase every linear gets a contiguous range of CTAs
// in proportion to its packed bytes and a CTA owns a contiguous range of 16-row groups of ONE linear, so
// it prepares one input vector per phase.  A CTA's (row unit, 256-column chunk) items are cut into one
// contiguous range per warp and streamed through a per-warp cp.async ring; partial sums meet in shared
// memory.  There is no device-wide barrier between the phases: every element of t is stored as one
// 64-bit {value, launch tag} word and phase 2 polls the elements it needs until they carry this launch's
// tag (nq_common.cuh); the poll is bounded and an expiry is sticky.  The launch is cooperative (consumers
// spin on data of CTAs that must be resident) with programmatic stream serialization: the descriptor
// reads, an L2 prefetch of ALL packed bytes this CTA will read in both phases, the first ring loads and
// the output scales run before griddepcontrol.wait, i.e. under the tail of the previous kernel, and the
// HBM stream of the factors overlaps the latency chain that follows.
//
// Everything a loop needs lives in registers: a shared-memory or parameter read behind an `asm volatile`
// with a memory clobber is re-issued every iteration.
//
// replaces: src/nanoquant/kernel/cuda/gemv_kernel.cu:43-301 of the reference
// (two kernels per linear, fp16/bf16 accumulation, sign-flip adds).
#include <cstring>

#include "nq_common.cuh"

namespace nq {

constexpr int kGemvThreads = 512;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxJobs = 4;         // linears per launch
constexpr int kMaxTok = 4;          // tokens per launch (3 byte terms each, 8 MMA columns per column group)
constexpr int kQMax = 64000;        // |X| bound: X * 2^7 splits into three signed bytes
constexpr int kMaxK = 32768;        // keeps sum(X) and every accumulator inside int32
#ifndef NQ_GEMV_STAGES
#define NQ_GEMV_STAGES 4
#endif
constexpr int kStages = NQ_GEMV_STAGES;          // 1 KB weight slots in flight per warp
constexpr size_t kStateBytes = 256;              // per-phase maxima, sums and units
constexpr size_t kRingBytes = (size_t)kGemvWarps * kStages * 1024;
constexpr size_t kHeaderBytes = 256;

// KIND_T: the rank-R intermediate between the phases, one 64-bit {fp32 value, launch tag} word per element
enum : int { KIND_F16 = 0, KIND_BF16 = 1, KIND_T = 2 };

#ifdef NQ_GEMV_TRACE  // development aid: per-warp (id, globaltimer, clock) records of the phase steps
__device__ unsigned long long g_trace[148 * 16 * 32 * 2];
__device__ __forceinline__ void trace_mark(int id) {
    __shared__ int s_n[16];
    if ((threadIdx.x & 31) == 0) {
        const int w = threadIdx.x >> 5;
        unsigned long long t, c;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(c));
        const int n = id == 0 ? 0 : s_n[w];
        if (n < 32) {
            unsigned long long* r = g_trace + ((size_t)(blockIdx.x * 16 + w) * 32 + n) * 2;
            r[0] = (t << 8) | (unsigned)id; r[1] = c;
            s_n[w] = n + 1;
            if (n + 1 < 32) r[2] = 0;
        }
    }
}
#define NQ_TRACE(id) trace_mark(id)
#else
#define NQ_TRACE(id) ((void)0)
#endif

// One linear in one phase.  Lives in the kernel parameters; every CTA reads the descriptor of the job it
// works on with uniform accesses into registers.
struct JobDesc {
    const uint4* tiles;   // [row_groups][chunks][32]
    const void* in;       // [T, ld_in] fp16/bf16 (phase 1) or tagged fp32 (phase 2)
    const void* pre;      // [K] scale in the I/O dtype, or nullptr
    const void* post;     // [rows] scale in the I/O dtype, or nullptr
    void* out;            // [T, ld_out] tagged fp32 (phase 1) or fp16/bf16 (phase 2)
    const void* bias;     // [rows] in the I/O dtype or nullptr (phase 2)
    const void* resid;    // [T, ld_res] in the I/O dtype or nullptr (phase 2)
    long long ld_in, ld_out, ld_res;
    int rows, K;
    int chunks;           // ceil(K / 256)
    int cta0, ncta;       // CTAs [cta0, cta0 + ncta) work on this job
    int rg_q, rg_r;       // 16-row groups per CTA: rg_q, one more for the first rg_r CTAs of the range
    int in_kind, out_kind;
    int vec;              // rows of `in` / `pre` are 16-byte aligned and K % 8 == 0
    int post_vec;         // `post` (and `bias`) 16-byte aligned and rows % 8 == 0: staged in shared memory
};

struct GemvParams {
    JobDesc job[2][kMaxJobs];
    unsigned* header;     // [0..1] 64-bit arrival counter (launch tags), [2] status
    int njobs;
    int T;
    int scale_kind;       // dtype of the scale vectors (KIND_F16 / KIND_BF16)
    int xq_stride;        // bytes between the int8 vectors in shared memory
    int rows_cap[2];      // most rows (16 per row group) a CTA owns in a phase
    unsigned spin_limit;  // polls before a wait for the tagged intermediate gives up
};

// The job descriptor fields the device code uses, in registers.
struct Work {
    const uint4* tiles;
    const void* in;
    const void* pre;
    const void* post;
    void* out;
    const void* bias;
    const void* resid;
    long long ld_in, ld_out, ld_res;
    int rows, K, chunks;
    int in_kind, out_kind, vec, post_vec;
    int rg0, cnt;         // this CTA's row groups: first, count (0: no work in this phase)
};

__device__ __forceinline__ float load_as_float(const void* p, long long i, int kind) {
    if (kind == KIND_F16) return __half2float(static_cast<const __half*>(p)[i]);
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight tagged elements (64 bytes) as floats, polled until all eight carry this launch's tag.
__device__ __forceinline__ void load8_tagged(const void* base, long long i, float (&v)[8], TagCtx& tc) {
    const unsigned long long* p = static_cast<const unsigned long long*>(base) + i;
    unsigned long long e[8];
    for (unsigned spins = 0;; ++spins) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
            asm volatile("ld.relaxed.gpu.global.v2.b64 {%0,%1}, [%2];"
                         : "=l"(e[2 * k]), "=l"(e[2 * k + 1]) : "l"(p + 2 * k) : "memory");
        bool ok = true;
#pragma unroll
        for (int k = 0; k < 8; ++k) ok = ok && (unsigned)(e[k] >> 32) == tc.tag;
        if (ok) break;
        if (spins >= tc.limit) { tag_wait_expired(tc); break; }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __uint_as_float((unsigned)e[k]);
}
__device__ __forceinline__ float load1_tagged(const void* base, long long i, TagCtx& tc) {
    const unsigned long long* p = static_cast<const unsigned long long*>(base) + i;
    unsigned long long e;
    for (unsigned spins = 0;; ++spins) {
        asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(e) : "l"(p) : "memory");
        if ((unsigned)(e >> 32) == tc.tag) break;
        if (spins >= tc.limit) { tag_wait_expired(tc); break; }
    }
    return __uint_as_float((unsigned)e);
}

// Eight consecutive 16-bit elements as floats.
template <int KIND>
__device__ __forceinline__ void to_float8(const uint4& u, float (&v)[8]) {
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

// Class-shifted operand of column k: X * 2^(7-j), negated for j = 7, j = (k % 256) / 32, as a multiplier.
__device__ __forceinline__ int class_mult(int j) { return (j == 7) ? -1 : (1 << (7 - j)); }

// Byte offset of column k inside an int8 vector: chunk base + 32*j + 8*q + 4*h + b for
// k % 256 = 32*j + 16*h + 4*q + b, so that lane (g, q) fetches the two B registers
// {k = 4q.., k = 16+4q..} of mask j with one 64-bit load.
__device__ __forceinline__ int xq_pos(int k) {
    const int kin = k & 255;
    return (k & ~255) + (kin & 0xE0) + 2 * (kin & 12) + ((kin & 16) >> 2) + (kin & 3);
}

// Units per value (0 when the maximum is zero, tiny or not finite: everything quantises to zero).
__device__ __forceinline__ float scale_from_max(float m, float& unit) {
    const bool good = (m > 1.0e-30f) && (m < 3.0e38f);
    unit = good ? m * (1.0f / (float)kQMax) : 0.f;
    // |p * inv| <= kQMax * (1 + 2^-21): the reciprocal is good to 1 ulp and the products round once each
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(m));
    return good ? (float)kQMax * r : 0.f;
}

// Z = Y + 0x808080 has the bytes b_t + 128 of the signed byte terms Y = b0 + 256 b1 + 65536 b2
// (|Y| < 2^23).  Four columns -> the three term words (column-major bytes), sign bit flipped back.
__device__ __forceinline__ void store_terms4(uint32_t z0, uint32_t z1, uint32_t z2, uint32_t z3, int8_t* dst,
                                             int stride) {
    const uint32_t t0 = __byte_perm(z0, z1, 0x5140), t1 = __byte_perm(z0, z1, 0x0062);
    const uint32_t t2 = __byte_perm(z2, z3, 0x5140), t3 = __byte_perm(z2, z3, 0x0062);
    *reinterpret_cast<uint32_t*>(dst) = __byte_perm(t0, t2, 0x5410) ^ 0x80808080u;
    *reinterpret_cast<uint32_t*>(dst + stride) = __byte_perm(t0, t2, 0x7632) ^ 0x80808080u;
    *reinterpret_cast<uint32_t*>(dst + 2 * stride) = __byte_perm(t1, t3, 0x5410) ^ 0x80808080u;
}

// Shared state of one phase (separate copies per phase: nothing has to be cleared between the jobs).
struct PhaseState {
    unsigned smax[kMaxTok];   // per-token max |input| as float bits (non-negative floats order like integers)
    int sumx[kMaxTok];        // per-token sum of the fixed-point values
    float unit[kMaxTok];      // value of one fixed-point unit
    unsigned pad[4];
};

// Eight columns of one token: products in, three byte vectors out; returns the sum of the fixed-point values.
__device__ __forceinline__ int convert8(const float (&p)[8], float inv, int k8, int8_t* row0, int stride) {
    const int mult = class_mult((k8 >> 5) & 7);
    uint32_t z[8];
    int acc = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int X = __float2int_rn(p[e] * inv);
        acc += X;
        z[e] = (uint32_t)(X * mult + 0x808080);
    }
    int8_t* dst = row0 + xq_pos(k8);
    store_terms4(z[0], z[1], z[2], z[3], dst, stride);
    store_terms4(z[4], z[5], z[6], z[7], dst + 8, stride);
    return acc;
}

// Quantise the input vectors of a job into shared memory.
//   xq: 3*T int8 vectors (row 3*tok + term, term 0 = least significant byte), `stride` bytes apart,
//       columns in xq_pos() order; columns K..Kpad are zero.
//   ps.sumx[tok]: sum of the (unshifted) fixed-point values, ps.unit[tok]: value of one unit.
// Register path: at most NB blocks of eight columns per thread; every value is loaded once, with all loads
// of the thread in flight together, and stays in registers between the max pass and the conversion.
// Block f = tid + i * threads covers token f / nv8, columns (f % nv8) * 8; nv8 is a multiple of 32, so a
// warp's block belongs to one token.
template <int IN_KIND, int NB>
__device__ __noinline__ void quantise_regs(const void* in, long long ld_in, const void* pre, int K, int chunks, int T,
                                           int8_t* xq, int stride, PhaseState* ps, TagCtx* tcp) {
    const int tid = threadIdx.x, lane = tid & 31;
    const int nv8 = chunks * 32, items = T * nv8;
    constexpr bool kHasPre = (IN_KIND != KIND_T);
    TagCtx tc = *tcp;
    float p[NB][8];
    int tt[NB], kk[NB];
    uint4 xr[NB], sr[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int f = tid + i * kGemvThreads;
        const int t = (f >= nv8) + (f >= 2 * nv8) + (f >= 3 * nv8);
        tt[i] = f < items ? t : -1;
        kk[i] = (f - t * nv8) * 8;
        xr[i] = sr[i] = make_uint4(0u, 0u, 0u, 0u);
        if (kHasPre && tt[i] >= 0 && kk[i] < K) {
            xr[i] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(in) + t * ld_in + kk[i]);
            sr[i] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(pre) + kk[i]));
        }
    }
    if (!tc.begun) tag_begin(tc, tc.status - 2, tc.limit);   // behind the input loads: the round trips overlap
    float wm[kMaxTok];   // this warp's maximum per token
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) wm[t] = 0.f;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        if (kHasPre) {
            float s[8];
            to_float8<IN_KIND>(xr[i], p[i]);
            to_float8<IN_KIND>(sr[i], s);
#pragma unroll
            for (int e = 0; e < 8; ++e) p[i][e] *= s[e];
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) p[i][e] = 0.f;
            if (tt[i] >= 0 && kk[i] < K) load8_tagged(in, tt[i] * ld_in + kk[i], p[i], tc);
        }
        float m = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(p[i][e]));
#pragma unroll
        for (int t = 0; t < kMaxTok; ++t) wm[t] = tt[i] == t ? fmaxf(wm[t], m) : wm[t];
    }
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) {
        if (t < T) {
            const unsigned r = __reduce_max_sync(0xffffffffu, __float_as_uint(wm[t]));
            if (lane == 0 && r != 0u) atomicMax(&ps->smax[t], r);
        }
    }
    asm volatile("" ::"r"(tc.tag));   // the tag has arrived in this thread before the CTA can arrive at the counter
    NQ_TRACE(2);
    __syncthreads();
    NQ_TRACE(3);
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        if (tt[i] >= 0) {      // warp-uniform
            float unit;
            const float inv = scale_from_max(__uint_as_float(ps->smax[tt[i]]), unit);
            if (kk[i] == 0) ps->unit[tt[i]] = unit;
            int acc = convert8(p[i], inv, kk[i], xq + (3 * tt[i]) * stride, stride);
            acc = __reduce_add_sync(0xffffffffu, acc);
            if (lane == 0 && acc != 0) atomicAdd(&ps->sumx[tt[i]], acc);
        }
    }
    *tcp = tc;
    NQ_TRACE(4);
    __syncthreads();
}

// Loop path for wider inputs (still 16-byte aligned rows, K % 8 == 0): two passes over the input, four blocks
// of a thread in flight; the second pass finds 16-bit inputs in L1 and the tagged intermediate valid.
template <int IN_KIND>
__device__ __noinline__ void quantise_loop(const void* in, long long ld_in, const void* pre, int K, int chunks, int T,
                                           int8_t* xq, int stride, PhaseState* ps, TagCtx* tcp) {
    const int tid = threadIdx.x, lane = tid & 31;
    const int Kpad = chunks * 256;
    constexpr bool kHasPre = (IN_KIND != KIND_T);
    constexpr int kBatch = 4;
    constexpr int kStep = kGemvThreads * 8;
    TagCtx tc = *tcp;
    if (!tc.begun) tag_begin(tc, tc.status - 2, tc.limit);
    auto load_products = [&](int t, int k0, float (&p)[kBatch][8]) {
        uint4 xr[kBatch], sr[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int k8 = k0 + u * kStep;
            xr[u] = sr[u] = make_uint4(0u, 0u, 0u, 0u);
            if (kHasPre && k8 < K) {
                xr[u] = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(in) + t * ld_in + k8);
                sr[u] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(pre) + k8));
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int k8 = k0 + u * kStep;
            if (kHasPre) {
                float s[8];
                to_float8<IN_KIND>(xr[u], p[u]);
                to_float8<IN_KIND>(sr[u], s);
#pragma unroll
                for (int e = 0; e < 8; ++e) p[u][e] *= s[e];
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) p[u][e] = 0.f;
                if (k8 < K) load8_tagged(in, t * ld_in + k8, p[u], tc);
            }
        }
    };
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float m = 0.f;
#pragma unroll 1
        for (int k0 = tid * 8; k0 < K; k0 += kStep * kBatch) {
            float p[kBatch][8];
            load_products(t, k0, p);
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
#pragma unroll
                for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(p[u][e]));
        }
        const unsigned r = __reduce_max_sync(0xffffffffu, __float_as_uint(m));
        if (lane == 0 && r != 0u) atomicMax(&ps->smax[t], r);
    }
    asm volatile("" ::"r"(tc.tag));
    NQ_TRACE(2);
    __syncthreads();
    NQ_TRACE(3);
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float unit;
        const float inv = scale_from_max(__uint_as_float(ps->smax[t]), unit);
        if (tid == 0) ps->unit[t] = unit;
        int acc = 0;
#pragma unroll 1
        for (int k0 = tid * 8; k0 < Kpad; k0 += kStep * kBatch) {
            float p[kBatch][8];
            load_products(t, k0, p);
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int k8 = k0 + u * kStep;
                if (k8 < Kpad) acc += convert8(p[u], inv, k8, xq + (3 * t) * stride, stride);   // columns K..Kpad are zero
            }
        }
        acc = __reduce_add_sync(0xffffffffu, acc);
        if (lane == 0 && acc != 0) atomicAdd(&ps->sumx[t], acc);
    }
    *tcp = tc;
    NQ_TRACE(4);
    __syncthreads();
}

// Scalar path for unaligned or ragged inputs (any K, any alignment).
__device__ __noinline__ void quantise_scalar(const void* in, long long ld_in, const void* pre, int K, int chunks, int T,
                                             int in_kind, int scale_kind, int8_t* xq, int stride, PhaseState* ps,
                                             TagCtx* tcp) {
    const int tid = threadIdx.x, lane = tid & 31;
    const int Kpad = chunks * 256;
    TagCtx tc = *tcp;
    if (!tc.begun) tag_begin(tc, tc.status - 2, tc.limit);
    auto product = [&](int t, int k) {
        const float s = pre ? load_as_float(pre, k, scale_kind) : 1.f;
        return (in_kind == KIND_T ? load1_tagged(in, t * ld_in + k, tc) : load_as_float(in, t * ld_in + k, in_kind)) * s;
    };
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float m = 0.f;
        for (int k = tid; k < K; k += kGemvThreads) m = fmaxf(m, fabsf(product(t, k)));
        const unsigned r = __reduce_max_sync(0xffffffffu, __float_as_uint(m));
        if (lane == 0 && r != 0u) atomicMax(&ps->smax[t], r);
    }
    asm volatile("" ::"r"(tc.tag));
    __syncthreads();
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float unit;
        const float inv = scale_from_max(__uint_as_float(ps->smax[t]), unit);
        if (tid == 0) ps->unit[t] = unit;
        int acc = 0;
        for (int k = tid; k < Kpad; k += kGemvThreads) {
            const int X = k < K ? __float2int_rn(product(t, k) * inv) : 0;
            acc += X;
            const uint32_t z = (uint32_t)(X * class_mult((k >> 5) & 7) + 0x808080) ^ 0x808080u;
            const int pos = xq_pos(k);
            xq[(3 * t) * stride + pos] = (int8_t)(z & 0xFF);
            xq[(3 * t + 1) * stride + pos] = (int8_t)((z >> 8) & 0xFF);
            xq[(3 * t + 2) * stride + pos] = (int8_t)((z >> 16) & 0xFF);
        }
        acc = __reduce_add_sync(0xffffffffu, acc);
        if (lane == 0 && acc != 0) atomicAdd(&ps->sumx[t], acc);
    }
    *tcp = tc;
    __syncthreads();
}

template <int NB>
__device__ __forceinline__ void quantise_regs_kind(const Work& w, int T, int8_t* xq, int stride, PhaseState* ps, TagCtx* tc) {
    if (w.in_kind == KIND_T) quantise_regs<KIND_T, NB>(w.in, w.ld_in, w.pre, w.K, w.chunks, T, xq, stride, ps, tc);
    else if (w.in_kind == KIND_F16) quantise_regs<KIND_F16, NB>(w.in, w.ld_in, w.pre, w.K, w.chunks, T, xq, stride, ps, tc);
    else quantise_regs<KIND_BF16, NB>(w.in, w.ld_in, w.pre, w.K, w.chunks, T, xq, stride, ps, tc);
}

__device__ __forceinline__ void quantise_input(const Work& w, int T, int scale_kind, int8_t* xq, int stride,
                                               PhaseState* ps, TagCtx* tc) {
    const int blocks = T * w.chunks * 32;
    if (!w.vec) quantise_scalar(w.in, w.ld_in, w.pre, w.K, w.chunks, T, w.in_kind, scale_kind, xq, stride, ps, tc);
    else if (blocks <= kGemvThreads) quantise_regs_kind<1>(w, T, xq, stride, ps, tc);
    else if (blocks <= 2 * kGemvThreads) quantise_regs_kind<2>(w, T, xq, stride, ps, tc);
    else if (blocks <= 4 * kGemvThreads) quantise_regs_kind<4>(w, T, xq, stride, ps, tc);
    else if (w.in_kind == KIND_T) quantise_loop<KIND_T>(w.in, w.ld_in, w.pre, w.K, w.chunks, T, xq, stride, ps, tc);
    else if (w.in_kind == KIND_F16) quantise_loop<KIND_F16>(w.in, w.ld_in, w.pre, w.K, w.chunks, T, xq, stride, ps, tc);
    else quantise_loop<KIND_BF16>(w.in, w.ld_in, w.pre, w.K, w.chunks, T, xq, stride, ps, tc);
}

__device__ __forceinline__ void cp_async16(unsigned smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Per-warp cursor over this warp's items of one job.  An item is one 256-column chunk of a row unit; a row
// unit is a pair of 16-row groups (tiles A and B, 1 KB together, sharing their B fragments) or, when a CTA
// has too few pairs to occupy its warps, a single group (tile B then repeats tile A and is discarded).
struct ItemStream {
    const uint4* next;    // tile A of the next item to fetch (this lane's 16 bytes)
    int offB;             // tile B of that item, in uint4, relative to tile A (0: none)
    int n_items;          // items of this warp
    int n_fetched;
    int f_c, f_ru;        // chunk and row unit of the next item to fetch
    int c0, ru0;          // chunk and row unit of this warp's first item
    int rpu;              // row groups per unit: 1 or 2
};

__device__ __forceinline__ void stream_issue(ItemStream& st, unsigned ring_lane, int chunks, int cnt) {
    if (st.n_fetched < st.n_items) {
        const unsigned dst = ring_lane + (unsigned)(st.n_fetched % kStages) * 1024u;
        cp_async16(dst, st.next);
        cp_async16(dst + 512u, st.next + st.offB);
        st.next += 32;
        ++st.n_fetched;
        if (++st.f_c == chunks) {      // next row unit: skip tile B's row group
            st.f_c = 0;
            ++st.f_ru;
            st.next += (st.rpu - 1) * chunks * 32;
            st.offB = (st.rpu == 2 && 2 * st.f_ru + 1 < cnt) ? chunks * 32 : 0;
        }
    }
    cp_async_commit();  // always commit so that group counting stays uniform
}

// Set the cursor up and start the first weight loads of a job.  They do not depend on the job's input
// vector, so this runs before the input is ready.
__device__ __forceinline__ void stream_begin(ItemStream& st, const Work& w, unsigned ring_lane, int warp, int lane) {
    const int pairs = (w.cnt + 1) >> 1;
    st.rpu = (pairs * w.chunks >= kGemvWarps) ? 2 : 1;
    const int units = st.rpu == 2 ? pairs : w.cnt;
    const int total = units * w.chunks;                       // < 2^20: the products below fit 32 bits
    const int begin = total * warp / kGemvWarps;
    st.n_items = total * (warp + 1) / kGemvWarps - begin;
    st.ru0 = 0;
    st.c0 = begin;
    while (st.c0 >= w.chunks) { st.c0 -= w.chunks; ++st.ru0; }   // at most `units` steps
    st.f_c = st.c0; st.f_ru = st.ru0; st.n_fetched = 0;
    st.next = w.tiles + ((size_t)(w.rg0 + st.ru0 * st.rpu) * w.chunks + st.c0) * 32 + lane;
    st.offB = (st.rpu == 2 && 2 * st.ru0 + 1 < w.cnt) ? w.chunks * 32 : 0;
#pragma unroll
    for (int d = 0; d < kStages - 1; ++d) stream_issue(st, ring_lane, w.chunks, w.cnt);
}

// The descriptor of the job this CTA works on in `phase` (cnt = 0: none), read with uniform accesses.
__device__ __forceinline__ void find_work(const GemvParams& P, int phase, Work& w) {
    w.cnt = 0;
    int sel = -1, rg0 = 0, cnt = 0;
#pragma unroll
    for (int j = 0; j < kMaxJobs; ++j) {
        if (j < P.njobs) {
            const JobDesc& J = P.job[phase][j];
            const int b = (int)blockIdx.x - J.cta0;
            if (b >= 0 && b < J.ncta) {
                sel = j;
                cnt = J.rg_q + (b < J.rg_r ? 1 : 0);
                rg0 = b * J.rg_q + min(b, J.rg_r);
            }
        }
    }
    if (sel < 0 || cnt == 0) return;
    const JobDesc& J = P.job[phase][sel];
    w.tiles = J.tiles; w.in = J.in; w.pre = J.pre; w.post = J.post; w.out = J.out; w.bias = J.bias; w.resid = J.resid;
    w.ld_in = J.ld_in; w.ld_out = J.ld_out; w.ld_res = J.ld_res;
    w.rows = J.rows; w.K = J.K; w.chunks = J.chunks;
    w.in_kind = J.in_kind; w.out_kind = J.out_kind; w.vec = J.vec; w.post_vec = J.post_vec;
    w.rg0 = rg0; w.cnt = cnt;
}

// Pull every packed byte this CTA will read in a phase towards L2 (bulk prefetches; the range is contiguous).
__device__ __forceinline__ void prefetch_tiles(const Work& w) {
    const char* p = reinterpret_cast<const char*>(w.tiles + (size_t)w.rg0 * w.chunks * 32);
    unsigned bytes = (unsigned)w.cnt * (unsigned)w.chunks * 512u;
    while (bytes > 0) {   // pieces well inside the instruction's size field
        const unsigned n = bytes > (1u << 20) ? (1u << 20) : bytes;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(n) : "memory");
        p += n;
        bytes -= n;
    }
}

// Output scales (and bias) of this CTA's rows into shared memory, as part of the thread's first copy group.
__device__ __forceinline__ void stage_row_vectors(const Work& w, uint16_t* post_s, uint16_t* bias_s) {
    if (!w.post_vec) return;
    const int row0 = 16 * w.rg0;
    const int nrows = min(16 * w.cnt, w.rows - row0);
    const int i = (int)threadIdx.x;
    if (8 * i < nrows) {
        if (w.post)
            cp_async16((unsigned)__cvta_generic_to_shared(post_s + 8 * i), static_cast<const uint16_t*>(w.post) + row0 + 8 * i);
        if (w.bias)
            cp_async16((unsigned)__cvta_generic_to_shared(bias_s + 8 * i), static_cast<const uint16_t*>(w.bias) + row0 + 8 * i);
    }
}

// The whole launch for one CTA: its job of phase 1, then its job of phase 2 (which polls the tagged
// intermediate).  CG = column groups of 8 MMA columns (3 columns per token).
template <int CG>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_group_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    constexpr int kCols = 8 * CG;
    NQ_TRACE(0);
    // shared memory carve-up
    PhaseState* pstate = reinterpret_cast<PhaseState*>(smem);                         // [2]
    const unsigned ring_lane = (unsigned)__cvta_generic_to_shared(smem + kStateBytes) +
                               (unsigned)warp * (kStages * 1024u) + (unsigned)lane * 16u;
    const uint4* ring_rd = reinterpret_cast<const uint4*>(smem + kStateBytes) + warp * (kStages * 64) + lane;
    int* s1_ph[2];
    s1_ph[0] = reinterpret_cast<int*>(smem + kStateBytes + kRingBytes);
    s1_ph[1] = s1_ph[0] + P.rows_cap[0] * kCols;
    int8_t* xq = reinterpret_cast<int8_t*>(s1_ph[1] + P.rows_cap[1] * kCols);
    uint16_t* post_ph[2];
    post_ph[0] = reinterpret_cast<uint16_t*>(xq + (size_t)3 * P.T * P.xq_stride);
    post_ph[1] = post_ph[0] + P.rows_cap[0];
    uint16_t* bias_s = post_ph[1] + P.rows_cap[1];

    Work wk[2];
    find_work(P, 0, wk[0]);
    find_work(P, 1, wk[1]);
    if (tid == 0 && wk[0].cnt > 0) prefetch_tiles(wk[0]);
    if (tid == 32 && wk[1].cnt > 0) prefetch_tiles(wk[1]);
    ItemStream st;
    st.n_items = 0;
    int ph = wk[0].cnt > 0 ? 0 : 1;
    if (wk[ph].cnt > 0) {
        stage_row_vectors(wk[ph], post_ph[ph], bias_s);
        stream_begin(st, wk[ph], ring_lane, warp, lane);
        // the input scales are constants of the layer: pull this thread's part towards L1 under the previous kernel's tail
        if (ph == 0 && wk[0].pre && tid * 8 < wk[0].K)
            asm volatile("prefetch.global.L1 [%0];" ::"l"(static_cast<const char*>(wk[0].pre) + 16 * (size_t)tid));
    }
    if (tid < (int)(2 * sizeof(PhaseState) / 4)) reinterpret_cast<unsigned*>(pstate)[tid] = 0u;
    for (int i = tid; i < (P.rows_cap[0] + P.rows_cap[1]) * kCols; i += kGemvThreads) s1_ph[0][i] = 0;
    __syncthreads();   // the zeroed state is in place before any warp can reach the atomics that use it
    NQ_TRACE(9);
    // Programmatic dependent launch: everything above may overlap with the tail of the previous kernel in the
    // stream; the activations and the scratch (shared with that kernel) are only touched after it has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // All CTAs of this cooperative grid are resident, so CTAs of the next kernel that start early cannot keep one
    // of ours from being scheduled: let the next kernel begin its prologue wherever an SM frees up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    NQ_TRACE(10);
    // tag of this launch for the intermediate's {value, tag} words
    TagCtx tc;
    tc.tag = 0u; tc.limit = P.spin_limit; tc.status = P.header + 2; tc.begun = 0u;   // read behind the first data loads
    bool arrived = false;

#pragma unroll 1
    for (; ph < 2; ++ph) {
        const Work& w = wk[ph];
        if (w.cnt == 0) continue;     // no rows of phase 2 for this CTA
        PhaseState* ps = pstate + ph;
        int* s1 = s1_ph[ph];
        quantise_input(w, P.T, P.scale_kind, xq, P.xq_stride, ps, &tc);
        if (!arrived) {   // behind a CTA barrier that every thread passes with its tag in hand
            if (tid == 0) launch_arrive(reinterpret_cast<unsigned long long*>(P.header), blockIdx.x == 0, gridDim.x);
            arrived = true;
        }
        NQ_TRACE(5);

        // MMA column n = 8*cg + g reads int8 vector n (= 3*tok + term); unused columns re-read a valid one
        const int ncols = 3 * P.T;
        const int8_t* bbase = xq + (g < ncols ? g : ncols - 1) * P.xq_stride + 8 * q;
        const int boff1 = CG > 1 ? ((8 + g < ncols ? 8 + g : ncols - 1) - (g < ncols ? g : ncols - 1)) * P.xq_stride : 0;
        const int chunks = w.chunks, cnt = w.cnt, n_items = st.n_items, rpu = st.rpu;
        int acc[2][2][CG][4];    // [tile A / B][even / odd mask: two independent MMA chains][column group][fragment]
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int cg = 0; cg < CG; ++cg)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[a][h][cg][i] = 0;
        int c_c = st.c0, c_ru = st.ru0;
#pragma unroll 1
        for (int n = 0; n < n_items; ++n) {
            stream_issue(st, ring_lane, chunks, cnt);
            cp_async_wait<kStages - 1>();
            // a lane reads back exactly the 32 bytes it copied itself: no warp synchronisation needed
            const uint4* slot = ring_rd + (n % kStages) * 64;
            const uint4 ta = slot[0], tb = slot[32];
            const int8_t* bp = bbase + c_c * 256;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t m = 0x01010101u << j;
#pragma unroll
                for (int cg = 0; cg < CG; ++cg) {
                    const uint2 b = *reinterpret_cast<const uint2*>(bp + (cg ? boff1 : 0) + 32 * j);
                    mma_s8(acc[0][j & 1][cg], ta.x & m, ta.y & m, ta.z & m, ta.w & m, b.x, b.y);
                    mma_s8(acc[1][j & 1][cg], tb.x & m, tb.y & m, tb.z & m, tb.w & m, b.x, b.y);
                }
            }
            // when this warp leaves the row unit, fold its partial sums into shared memory:
            // lane (g, q) holds rows g / g+8 of both tiles, columns 2q, 2q+1 of each column group
            if (++c_c == chunks || n + 1 == n_items) {
                int* dst = s1 + c_ru * rpu * (16 * kCols);
                const bool has_b = rpu == 2 && 2 * c_ru + 1 < cnt;
#pragma unroll
                for (int cg = 0; cg < CG; ++cg) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int col = 8 * cg + 2 * q + (i & 1);
                        const int ra = g + 8 * (i >> 1);
                        const int va = acc[0][0][cg][i] + acc[0][1][cg][i];
                        const int vb = acc[1][0][cg][i] + acc[1][1][cg][i];
                        if (col < ncols) {
                            if (va != 0) atomicAdd(&dst[ra * kCols + col], va);
                            if (has_b && vb != 0) atomicAdd(&dst[(16 + ra) * kCols + col], vb);
                        }
                        acc[0][0][cg][i] = 0; acc[0][1][cg][i] = 0;
                        acc[1][0][cg][i] = 0; acc[1][1][cg][i] = 0;
                    }
                }
                if (c_c == chunks) { c_c = 0; ++c_ru; }
            }
        }
        cp_async_wait<0>();
        NQ_TRACE(11);
        // This warp's ring is free again (a lane only ever reads its own bytes): start the weight stream and the
        // output scales of the phase-2 job before the barrier and the epilogue, whose latencies the loads overlap.
        if (ph == 0 && wk[1].cnt > 0) {
            stage_row_vectors(wk[1], post_ph[1], bias_s);
            stream_begin(st, wk[1], ring_lane, warp, lane);
        }
        __syncthreads();
        NQ_TRACE(6);
        // finalise: the three column sums of a token are the byte terms of 128 * sum_{bit=1}(X);
        // result = sum(X) - 2 * sum_{bit=1}(X) = sum(X) - terms / 64 (terms is a multiple of 128).
        const int row0 = 16 * w.rg0;
        const int nrows = min(16 * cnt, w.rows - row0);
        const uint16_t* my_post = post_ph[ph];
#pragma unroll 1
        for (int tok = 0; tok < P.T; ++tok) {
            const long long sx = ps->sumx[tok];
            const float unit = ps->unit[tok];
#pragma unroll 1
            for (int idx = tid; idx < nrows; idx += kGemvThreads) {
                const int row = row0 + idx;
                float extra = 0.f;       // bias and residual of this output, fetched before the arithmetic
                if (w.bias) extra = w.post_vec ? load_as_float(bias_s, idx, P.scale_kind) : load_as_float(w.bias, row, P.scale_kind);
                if (w.resid) extra += load_as_float(w.resid, tok * w.ld_res + row, P.scale_kind);
                const int* c = s1 + idx * kCols + 3 * tok;
                const long long terms = (long long)c[2] * 65536 + (long long)c[1] * 256 + (long long)c[0];
                const long long r = sx - (terms >> 6);
                // exact split: both halves convert without rounding, the sum rounds once
                float val = ((float)(int)(r >> 20) * 1048576.0f + (float)(int)(r & 0xFFFFF)) * unit;
                if (w.post) val *= w.post_vec ? load_as_float(my_post, idx, P.scale_kind) : load_as_float(w.post, row, P.scale_kind);
                if (w.out_kind == KIND_T) {
                    store_tagged(w.out, tok * w.ld_out + row, val, tc.tag);
                } else {
                    val += extra;
                    if (w.out_kind == KIND_F16) {
                        // same saturation bounds as the reference epilogue
                        val = fminf(fmaxf(val, -64504.0f), 64504.0f);
                        static_cast<__half*>(w.out)[tok * w.ld_out + row] = __float2half(val);
                    } else {
                        val = fminf(fmaxf(val, -3.3895313892515355e+38f), 3.3895313892515355e+38f);
                        static_cast<__nv_bfloat16*>(w.out)[tok * w.ld_out + row] = __float2bfloat16(val);
                    }
                }
            }
        }
        NQ_TRACE(12);
    }
    if (!arrived) {   // a CTA without rows in either phase still counts towards the launch
        if (!tc.begun) tag_begin(tc, tc.status - 2, tc.limit);
        asm volatile("" ::"r"(tc.tag));
        __syncthreads();
        if (tid == 0) launch_arrive(reinterpret_cast<unsigned long long*>(P.header), blockIdx.x == 0, gridDim.x);
    }
}

static size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

// Opt-in shared memory limit for both instantiations, set once per device.
static int dynamic_smem_limit(int dev, int* out) {
    static int cached[64];
    if (cached[dev & 63] == 0) {
        int optin = 0, lim = 1 << 30;
        NQ_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        const void* fns[2] = {(const void*)gemv_group_kernel<1>, (const void*)gemv_group_kernel<2>};
        for (const void* fn : fns) {
            cudaFuncAttributes fa;
            NQ_CUDA_TRY(cudaFuncGetAttributes(&fa, fn));
            const int v = optin - (int)fa.sharedSizeBytes;  // the opt-in limit covers static + dynamic
            NQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
            lim = v < lim ? v : lim;
        }
        cached[dev & 63] = lim;
    }
    *out = cached[dev & 63];
    return NQ_OK;
}

// Deal the CTAs of the grid to the jobs of a phase: every job gets a contiguous range, sized so that the
// longest per-CTA stream (row groups x chunks) is as short as possible; a CTA never owns rows of two jobs.
// Returns the most row groups a CTA owns.
static int plan_phase(JobDesc* jobs, int njobs, int grid) {
    int rg[kMaxJobs], n[kMaxJobs];
    for (int j = 0; j < njobs; ++j) {
        rg[j] = (jobs[j].rows + 15) / 16;
        n[j] = 1;
    }
    for (int used = njobs; used < grid; ++used) {
        int best = -1;
        long long best_cost = -1;
        for (int j = 0; j < njobs; ++j) {
            if (n[j] >= rg[j]) continue;      // one row group per CTA already
            const long long cost = (long long)((rg[j] + n[j] - 1) / n[j]) * jobs[j].chunks;
            if (cost > best_cost) { best_cost = cost; best = j; }
        }
        if (best < 0) break;
        ++n[best];
    }
    int c0 = 0, cap = 0;
    for (int j = 0; j < njobs; ++j) {
        jobs[j].cta0 = c0;
        jobs[j].ncta = n[j];
        jobs[j].rg_q = rg[j] / n[j];
        jobs[j].rg_r = rg[j] % n[j];
        const int most = jobs[j].rg_q + (jobs[j].rg_r ? 1 : 0);
        cap = most > cap ? most : cap;
        c0 += n[j];
    }
    return cap;
}

// ---------------------------------------------------------------------------
// GEMV without caller-provided scratch
// ---------------------------------------------------------------------------
// Scratch of nq_gemv_fwd_static: lives in the library image on every GPU that loads it, until
// the process exits.  256-byte header + tagged fp32 intermediate (8 bytes per element) for up to 4 tokens x rank 8192.
constexpr int kStaticMaxRank = 8192;
constexpr size_t kStaticScratchBytes = kHeaderBytes + (size_t)kMaxTok * kStaticMaxRank * sizeof(uint2);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the symbol name is
// only a handle: the address a kernel can use comes from cudaGetSymbolAddress, looked up once
// per device with that device current.  The cached address stays valid as long as the device's
// primary context is not reset.
static int static_scratch_ptr(void** out) {
    static void* cached[64];
    int dev = 0;
    NQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NQ_ERR_UNSUPPORTED;
    if (!cached[dev]) {
        void* p = nullptr;
        NQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return NQ_ERR_CUDA;
        cached[dev] = p;
    }
    *out = cached[dev];
    return NQ_OK;
}

static unsigned g_spin_limit = kSpinLimit;

}  // namespace nq

using namespace nq;

extern "C" {

size_t nq_gemv_scratch_bytes(int T, int N, int R, int M) {
    if (T <= 0 || N <= 0 || R <= 0 || M <= 0) return 0;
    return kHeaderBytes + round_up((size_t)kMaxTok * (size_t)R * sizeof(uint2), 256);
}

size_t nq_gemv_group_scratch_bytes(const nq_linear_desc* d, int n_linears, int T) {
    if (!d || n_linears <= 0 || n_linears > kMaxJobs || T <= 0) return 0;
    size_t b = kHeaderBytes;
    for (int i = 0; i < n_linears; ++i) {
        if (d[i].R <= 0) return 0;
        b += round_up((size_t)kMaxTok * (size_t)d[i].R * sizeof(uint2), 256);
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
        if (L.residual && L.ldr < L.M) return NQ_ERR_SHAPE;
        if (L.N > kMaxK || L.R > kMaxK) return NQ_ERR_UNSUPPORTED;
        if (!aligned16(L.v_tiles) || !aligned16(L.u_tiles)) return NQ_ERR_ALIGN;
        maxK = L.N > maxK ? L.N : maxK;
        maxK = L.R > maxK ? L.R : maxK;
    }
    int dev = 0, smem_limit = 0;
    NQ_CUDA_TRY(cudaGetDevice(&dev));
    {
        const int st = dynamic_smem_limit(dev, &smem_limit);
        if (st != NQ_OK) return st;
    }
    const int grid = sm_count();
    if (grid < kMaxJobs || (unsigned)grid >= kTagSpan) return NQ_ERR_UNSUPPORTED;
    const int kpad = (maxK + 255) / 256 * 256;
    const int stride = kpad + 32;  // 32 mod 128: conflict-free 64-bit fragment loads

    GemvParams P;
    memset(&P, 0, sizeof(P));
    P.header = static_cast<unsigned*>(scratch);
    P.scale_kind = dtype;
    P.xq_stride = stride;
    P.njobs = n_linears;
    P.spin_limit = g_spin_limit;
    const size_t esz = 2;
    size_t off = kHeaderBytes;
    for (int i = 0; i < n_linears; ++i) {
        const nq_linear_desc& L = d[i];
        void* tbuf = static_cast<char*>(scratch) + off;   // {fp32, tag} words, 8 bytes per element
        off += round_up((size_t)kMaxTok * (size_t)L.R * sizeof(uint2), 256);
        JobDesc& a = P.job[0][i];
        a.tiles = static_cast<const uint4*>(L.v_tiles);
        a.in = L.x;
        a.pre = L.s_in;
        a.post = L.s_mid;
        a.out = tbuf;
        a.ld_in = L.ldx;
        a.ld_out = L.R;
        a.rows = L.R;
        a.K = L.N;
        a.chunks = (L.N + 255) / 256;
        a.in_kind = dtype;
        a.out_kind = KIND_T;
        a.post_vec = L.s_mid && (L.R % 8 == 0) && aligned16(L.s_mid);
        JobDesc& b = P.job[1][i];
        b.tiles = static_cast<const uint4*>(L.u_tiles);
        b.in = tbuf;
        b.post = L.s_out;
        b.out = L.y;
        b.bias = L.bias;
        b.resid = L.residual;
        b.ld_in = L.R;
        b.ld_out = L.ldy;
        b.ld_res = L.ldr;
        b.rows = L.M;
        b.K = L.R;
        b.chunks = (L.R + 255) / 256;
        b.in_kind = KIND_T;
        b.out_kind = dtype;
        b.vec = (L.R % 8 == 0);  // the intermediate lives in the 256-byte aligned scratch
        b.post_vec = (L.M % 8 == 0) && aligned16(L.s_out) && (!L.bias || aligned16(L.bias));
    }
    for (int ph = 0; ph < 2; ++ph) P.rows_cap[ph] = 16 * plan_phase(P.job[ph], n_linears, grid);

    // tokens are processed in groups that fit the MMA columns (3 per token) and shared memory
    auto cg_for = [](int t) { return t <= 2 ? 1 : 2; };
    auto smem_for = [&](int t) {
        const size_t rows = (size_t)P.rows_cap[0] + P.rows_cap[1];
        return kStateBytes + kRingBytes + rows * (32 * cg_for(t)) + (size_t)3 * t * stride +
               round_up(rows * 2, 16) + round_up((size_t)P.rows_cap[1] * 2, 16) + 32;
    };
    int tg = T < kMaxTok ? T : kMaxTok;
    while (tg > 1 && smem_for(tg) > (size_t)smem_limit) --tg;
    if (smem_for(tg) > (size_t)smem_limit) return NQ_ERR_UNSUPPORTED;

    for (int t0 = 0; t0 < T; t0 += tg) {
        const int tn = (T - t0) < tg ? (T - t0) : tg;
        P.T = tn;
        for (int i = 0; i < n_linears; ++i) {
            const nq_linear_desc& L = d[i];
            P.job[0][i].in = static_cast<const char*>(L.x) + (size_t)t0 * L.ldx * esz;
            P.job[0][i].vec = (L.N % 8 == 0) && (L.ldx % 8 == 0) && aligned16(P.job[0][i].in) && aligned16(L.s_in);
            P.job[1][i].out = static_cast<char*>(L.y) + (size_t)t0 * L.ldy * esz;
            if (L.residual) P.job[1][i].resid = static_cast<const char*>(L.residual) + (size_t)t0 * L.ldr * esz;
        }
        void* args[] = {&P};
        const void* fn = cg_for(tn) == 1 ? (const void*)gemv_group_kernel<1> : (const void*)gemv_group_kernel<2>;
        // Cooperative launch (all CTAs co-resident: phase 2 spins on data of other CTAs) plus programmatic stream
        // serialization, so that this kernel's prologue overlaps the previous kernel's tail.  If the driver
        // refuses the combination once, plain cooperative launches are used from then on.
        static bool pdl_ok = true;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kGemvThreads);
        cfg.dynamicSmemBytes = smem_for(tn);
        cfg.stream = as_stream(stream);
        cudaLaunchAttribute attrs[2];
        attrs[0].id = cudaLaunchAttributeCooperative;
        attrs[0].val.cooperative = 1;
        attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attrs;
        cfg.numAttrs = pdl_ok ? 2 : 1;
        cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
        if (e != cudaSuccess && pdl_ok) {
            (void)cudaGetLastError();
            pdl_ok = false;
            cfg.numAttrs = 1;
            e = cudaLaunchKernelExC(&cfg, fn, args);
        }
        NQ_CUDA_TRY(e);
    }
    return NQ_OK;
}

int nq_gemv_fwd(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                const void* u_tiles, const void* s_out, void* y, void* scratch, size_t scratch_bytes,
                int T, int N, int R, int M, int dtype, nq_stream_t stream) {
    nq_linear_desc d;
    memset(&d, 0, sizeof(d));
    d.x = x; d.s_in = s_in; d.v_tiles = v_tiles; d.s_mid = s_mid; d.u_tiles = u_tiles; d.s_out = s_out;
    d.y = y; d.N = N; d.R = R; d.M = M; d.ldx = N; d.ldy = M;
    return nq_gemv_group_fwd(&d, 1, T, dtype, scratch, scratch_bytes, stream);
}

int nq_gemv_fwd_static(const void* x, const void* s_in, const void* v_tiles, const void* s_mid,
                       const void* u_tiles, const void* s_out, void* y,
                       int T, int N, int R, int M, int dtype, nq_stream_t stream) {
    if (T <= 0 || N <= 0 || R <= 0 || M <= 0) return NQ_ERR_SHAPE;
    if (R > kStaticMaxRank || nq_gemv_scratch_bytes(T, N, R, M) > kStaticScratchBytes) return NQ_ERR_TOO_LARGE;
    void* scratch = nullptr;
    const int st = static_scratch_ptr(&scratch);   // first call on a device: symbol lookup
    if (st != NQ_OK) return st;
    // Nothing has to be cleared between calls: the array is zero when the library is loaded, the arrival
    // counter in its header runs freely (every launch derives a fresh tag from it) and stale intermediate
    // elements carry older tags.
    return nq_gemv_fwd(x, s_in, v_tiles, s_mid, u_tiles, s_out, y, scratch, kStaticScratchBytes, T, N, R, M, dtype,
                       stream);
}

size_t nq_gemv_static_max_rank(void) { return (size_t)kStaticMaxRank; }

#ifdef NQ_GEMV_TRACE
int nq_debug_read_trace(unsigned long long* host_out) {
    NQ_CUDA_TRY(cudaDeviceSynchronize());
    NQ_CUDA_TRY(cudaMemcpyFromSymbol(host_out, g_trace, sizeof(unsigned long long) * 148 * 16 * 32 * 2));
    return NQ_OK;
}
#endif

unsigned nq_gemv_set_wait_limit(unsigned polls) {
    const unsigned old = g_spin_limit;
    g_spin_limit = polls ? polls : kSpinLimit;
    return old;
}

int nq_scratch_status(const void* scratch, nq_stream_t stream) {
    if (!scratch) {   // the array of nq_gemv_fwd_static
        void* p = nullptr;
        const int st = static_scratch_ptr(&p);
        if (st != NQ_OK) return st;
        scratch = p;
    }
    unsigned h[4] = {0, 0, 0, 0};
    NQ_CUDA_TRY(cudaMemcpyAsync(h, scratch, sizeof(h), cudaMemcpyDeviceToHost, as_stream(stream)));
    NQ_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    return h[2] == 0 ? NQ_OK : -(int)h[2];
}

}  // extern "C"
