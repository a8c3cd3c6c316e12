// Decode GEMV for the binary low-rank linear, one launch per group of linears.
//
//   y = s_out * (U . (s_mid * (V . (s_in * x))))          T <= 4 tokens per launch
//
// The kernel is bound by the HBM stream of the packed factors and, for the layer
// sizes of 8B-class decoders, by latency; both call for as few instructions per
// weight and per phase as possible.
//
//  * The packed sign bits are the A operand of an integer tensor-core MMA
//    (mma.sync m16n8k32 s8*s8->s32) WITHOUT unpacking: in the tile layout (see
//    nq_rows_to_tiles) `word & (0x01010101 << j)` is an int8x4 register with values
//    {0, 2^j} ({0, -128} for j = 7), so one LOP3 prepares four weights and the eight
//    masks j = 0..7 consume a whole 32-bit word.  Columns [32j, 32j+32) of a
//    256-column chunk form the "class" j.
//  * The input vector of a phase (s_in*x, or the rank-R intermediate t) is turned,
//    once per CTA, into 17-bit fixed point X with a per-token scale.  A column of
//    class j is stored as X * 2^(7-j) (negated for j = 7), split into three signed
//    bytes.  The product of the A value 2^j and that operand is 2^7 * X for every
//    class, so all eight masks accumulate into ONE accumulator per output row and
//    byte term.  The three byte terms of a token are three of the N = 8 MMA columns.
//  * sum(+-X) = sum(X) - 2 * sum_{bit=1}(X).  All accumulation is exact int32 /
//    int64, so the result does not depend on the order in which warps add up.
//
// A SIMT sign-flip-add inner loop issues ~1.5 instructions per weight and tops out
// near one third of the HBM rate on this part, which is why the integer MMA is
// used as a wide dot-product unit here.
//
// Phases: phase 1 computes t[T,R] (fp32, in scratch), phase 2 computes y.  Several
// linears that share the two phases (q/k/v, gate/up) are processed in one launch.
// There is no device-wide barrier between the phases: every element of t is stored
// together with a tag of the launch and phase 2 polls the elements it needs until
// they carry this launch's tag (see tag_begin / load8_tagged); the poll is bounded:
// on expiry a status word is set and the thread goes on.  The weight stream of the
// next job is started before that wait, so it overlaps with HBM traffic.  The kernel
// is launched cooperative (all CTAs resident: consumers spin on other CTAs' data) and
// with programmatic stream serialization: everything that does not depend on the
// previous kernel (descriptor copy, first weight loads, an L2 prefetch of the input
// scales) runs before griddepcontrol.wait.
//
// For 8B-class layers the kernel is a chain of dependent latencies (memory round
// trips, CTA barriers, the hand-over of t between the phases), not a bandwidth problem; the code
// between the main loops is therefore kept short and free of divisions.
//
// replaces: src/nanoquant/kernel/cuda/gemv_kernel.cu:43-301 of the reference
// (two kernels per linear, fp16/bf16 accumulation, sign-flip adds).
#include <cstring>

#include "nq_common.cuh"

namespace nq {

#ifndef NQ_GEMV_THREADS
#define NQ_GEMV_THREADS 512
#endif
#ifndef NQ_GEMV_STAGES
#define NQ_GEMV_STAGES 4
#endif
#ifndef NQ_GEMV_MIN_CTAS
#define NQ_GEMV_MIN_CTAS 1
#endif
constexpr int kGemvThreads = NQ_GEMV_THREADS;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxJobs = 4;         // linears per launch
constexpr int kMaxTok = 4;          // tokens per launch (3 byte terms each, 8 MMA columns per column group)
constexpr int kQMax = 64000;        // |X| bound: X * 2^7 splits into three signed bytes
constexpr int kMaxK = 32768;        // keeps sum(X) and every accumulator inside int32
constexpr int kStages = NQ_GEMV_STAGES;          // 1 KB weight slots in flight per warp
constexpr size_t kRedBytes = 384;   // per-warp maxima: kMaxTok * kGemvWarps floats (16-byte aligned rows)
constexpr size_t kFixedBytes = 512;
constexpr size_t kRingBytes = (size_t)kGemvWarps * kStages * 1024;
constexpr size_t kHeaderBytes = 256;
constexpr unsigned kPollBackoffNs = 200;   // pause between two polls of the tagged intermediate

// KIND_T: the rank-R intermediate between the phases, one 8-byte {fp32 value, launch tag} pair per element
enum : int { KIND_F16 = 0, KIND_BF16 = 1, KIND_T = 2 };

struct Job {
    const uint4* tiles;   // [row_groups][chunks][32]
    const void* in;       // [T, ld_in]  fp16/bf16 (phase 1) or fp32 (phase 2)
    const void* pre;      // [K] scale in the I/O dtype, or nullptr
    const void* post;     // [rows] scale in the I/O dtype, or nullptr
    void* out;            // [T, ld_out] fp32 (phase 1) or fp16/bf16 (phase 2)
    const void* bias;     // [rows] in the I/O dtype or nullptr (phase 2)
    const void* resid;    // [T, ld_res] in the I/O dtype or nullptr (phase 2)
    long long ld_in, ld_out, ld_res;
    int rows, K;
    int chunks;           // ceil(K / 256)
    int items;            // ceil(rows / 32)
    int in_kind, out_kind;
    int vec;              // rows of `in` / `pre` are 16-byte aligned and K % 8 == 0
    int cta0, ncta;       // CTAs [cta0, cta0 + ncta) work on this job
    int t_q, t_r;         // row tiles per CTA of the range: t_q, one more for its first t_r CTAs
    int post_vec;         // `post` is 16-byte aligned and rows % 8 == 0: staged in shared memory with 16-byte copies
};

struct Phase {
    Job job[kMaxJobs];
    int njobs;
};

struct GemvParams {
    Phase phase[2];
    unsigned* header;     // [0..1] 64-bit arrival counter (launch tags), [2] status
    unsigned spin_limit;  // polls before a wait for the tagged intermediate gives up
    int T;
    int scale_kind;       // dtype of the scale vectors (KIND_F16 / KIND_BF16)
    int xq_stride;        // bytes between the int8 vectors in shared memory
    int max_items;        // row tiles a CTA may own per job
};

__device__ __forceinline__ float load_as_float(const void* p, long long i, int kind) {
    if (kind == KIND_F16) return __half2float(static_cast<const __half*>(p)[i]);
    if (kind == KIND_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return 0.f;   // the tagged intermediate goes through load1_tagged / load8_tagged
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight tagged elements (64 bytes) as floats, polled until all eight carry this launch's tag.  Every element is
// one 64-bit word {value, tag}: a 64-bit access is single-copy atomic, so a matching tag implies its value.
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
        __nanosleep(kPollBackoffNs);   // failed polls of 148 CTAs load the L2 lines the producers are storing to
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

// Eight consecutive elements of a vector as floats (one or two 128-bit loads).
template <int KIND>
__device__ __forceinline__ void load8(const void* base, long long i, float (&v)[8], TagCtx& tc) {
    if (KIND == KIND_T) {
        load8_tagged(base, i, v, tc);
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

// The launch tag is read behind the first input loads of the kernel (see tag_begin).
__device__ __forceinline__ void tag_ensure(TagCtx& tc) {
    if (!tc.begun) tag_begin(tc, tc.status - 2, tc.limit);
}


// The same split in two: the raw 128-bit loads of a block (so that several blocks can be in flight before
// the first conversion) and the conversion.
template <int KIND>
struct Raw8 { uint4 a, b; };   // b: second half of an fp32 block
template <int KIND>
__device__ __forceinline__ void load_raw(const void* base, long long i, Raw8<KIND>& r, TagCtx& tc) {
    if (KIND == KIND_T) {   // tagged pairs are polled until valid; the block keeps the eight values
        float v[8];
        load8_tagged(base, i, v, tc);
        r.a = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
        r.b = make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7]));
    } else {
        r.a = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + i);
    }
}
template <int KIND>
__device__ __forceinline__ void to_float8(const Raw8<KIND>& r, float (&v)[8]) {
    if (KIND == KIND_T) {
        v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y); v[2] = __uint_as_float(r.a.z); v[3] = __uint_as_float(r.a.w);
        v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y); v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
    } else {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (KIND == KIND_F16) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                v[2 * e] = f.x; v[2 * e + 1] = f.y;
            } else {
                v[2 * e] = __uint_as_float(w[e] << 16);
                v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
            }
        }
    }
}

// Class-shifted operand of column k: X * 2^(7-j), negated for j = 7, j = (k % 256) / 32.
__device__ __forceinline__ int class_shift(int X, int j) { return (j == 7) ? -X : (X << (7 - j)); }

// Byte offset of column k inside an int8 vector: chunk base + 32*j + 8*q + 4*h + b for
// k % 256 = 32*j + 16*h + 4*q + b, so that lane (g, q) fetches the two B registers
// {k = 4q.., k = 16+4q..} of mask j with one 64-bit load.
__device__ __forceinline__ int xq_pos(int k) {
    const int kin = k & 255;
    return (k & ~255) + (kin & 0xE0) + 2 * (kin & 12) + ((kin & 16) >> 2) + (kin & 3);
}

// red[t * kGemvWarps + warp] holds the per-warp maxima of token t.  Every thread derives the fixed-point
// scale of its token from them itself (a few broadcast reads), which saves a serial step and a CTA barrier.
__device__ __forceinline__ float token_max(const float* red, int t) {
    const float4* r = reinterpret_cast<const float4*>(red + t * kGemvWarps);
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < kGemvWarps / 4; ++i) {
        const float4 v = r[i];
        m = fmaxf(m, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
    return m;
}
// Units per value (0 when the maximum is zero or not finite: everything quantises to zero); the thread
// for which `writer` holds records the value of one unit for the epilogue.
__device__ __forceinline__ float token_inv(const float* red, int t, bool writer, float* delta) {
    const float m = token_max(red, t);
    const bool good = (m > 0.f) && (m < 3.0e38f);
    // A rounded reciprocal times kQMax instead of a division: every thread computes the same value,
    // |p * inv| stays within kQMax (1 + 2^-22), and the unit differs from 1 / inv by a relative 2^-22 at most.
    if (writer) delta[t] = good ? m * (1.0f / (float)kQMax) : 0.f;
    return good ? (float)kQMax * __frcp_rn(m) : 0.f;
}
// Warp-wide maximum of non-negative floats / sum of ints with one reduction instruction each.
__device__ __forceinline__ float warp_max_abs(float m) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
}

// Write eight class-shifted operands (columns k8..k8+7 of one token) as three byte vectors.
__device__ __forceinline__ void store_terms(const uint32_t (&Y)[8], int8_t* r0, int stride, int k8) {
    // Y = 65536*b2 + 256*b1 + b0 with signed bytes: b0 = byte 0 of Y, b1 = byte 1 of
    // Y + 0x80, b2 = byte 2 of Y + 0x8080
    const int pos = xq_pos(k8);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        const uint32_t y0 = Y[4 * w], y1 = Y[4 * w + 1], y2 = Y[4 * w + 2], y3 = Y[4 * w + 3];
        const uint32_t z0 = y0 + 0x80u, z1 = y1 + 0x80u, z2 = y2 + 0x80u, z3 = y3 + 0x80u;
        const uint32_t u0 = y0 + 0x8080u, u1 = y1 + 0x8080u, u2 = y2 + 0x8080u, u3 = y3 + 0x8080u;
        const uint32_t b0 = __byte_perm(__byte_perm(y0, y1, 0x0040), __byte_perm(y2, y3, 0x0040), 0x5410);
        const uint32_t b1 = __byte_perm(__byte_perm(z0, z1, 0x0051), __byte_perm(z2, z3, 0x0051), 0x5410);
        const uint32_t b2 = __byte_perm(__byte_perm(u0, u1, 0x0062), __byte_perm(u2, u3, 0x0062), 0x5410);
        *reinterpret_cast<uint32_t*>(r0 + pos + 8 * w) = b0;
        *reinterpret_cast<uint32_t*>(r0 + stride + pos + 8 * w) = b1;
        *reinterpret_cast<uint32_t*>(r0 + 2 * stride + pos + 8 * w) = b2;
    }
}

// Quantise the input vectors of a job into shared memory.
//   xq: 3*T int8 vectors (row 3*tok + term, term 0 = least significant byte), `stride`
//       bytes apart, columns in xq_pos() order; columns K..Kpad are zero.
//   sumx[tok]: sum of the (unshifted) fixed-point values, delta[tok]: value of one unit.
// The code is kept as small loops on purpose: it runs once per phase, where
// instruction fetch and latency, not arithmetic, set the pace.
//
// Vector path: rows of `in` / `pre` 16-byte aligned, K % 8 == 0; eight columns per thread and step.
template <int IN_KIND>
__device__ __noinline__ void quantise_vec(const Job& jb, int T, int8_t* xq, int stride, float* red,
                                          int* sumx, float* delta, TagCtx& tc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, Kpad = jb.chunks * 256;
    constexpr bool kHasPre = (IN_KIND != KIND_T);
    constexpr int kBatch = 4;                       // blocks whose loads are issued before the first use:
    constexpr int kStep = kGemvThreads * 8;         // one memory round trip per batch instead of one per block
    tag_ensure(tc);
    // pass 1: per-token max |in * pre|
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float m = 0.f;
#pragma unroll 1
        for (int k0 = tid * 8; k0 < K; k0 += kStep * kBatch) {
            Raw8<IN_KIND> x[kBatch], sc[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int k8 = k0 + u * kStep;
                x[u].a = x[u].b = make_uint4(0u, 0u, 0u, 0u);     // a zero block does not move the maximum
                sc[u].a = sc[u].b = make_uint4(0u, 0u, 0u, 0u);
                if (k8 < K) {
                    load_raw<IN_KIND>(jb.in, t * jb.ld_in + k8, x[u], tc);
                    if (kHasPre) load_raw<IN_KIND>(jb.pre, k8, sc[u], tc);
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                float v[8], s[8];
                to_float8<IN_KIND>(x[u], v);
                if (kHasPre) to_float8<IN_KIND>(sc[u], s);
#pragma unroll
                for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(kHasPre ? v[e] * s[e] : v[e]));
            }
        }
        m = warp_max_abs(m);
        if (lane == 0) red[t * kGemvWarps + warp] = m;
    }
    if (tid < kMaxTok) sumx[tid] = 0;
    asm volatile("" ::"r"(tc.tag));   // the tag is in this thread's hands before the CTA can arrive at the counter
    __syncthreads();
    // pass 2: |p * inv| <= kQMax + 2^-7 by construction (same products as in pass 1), no clamp needed
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float inv = token_inv(red, t, tid == 0, delta);
        int8_t* r0 = xq + (3 * t) * stride;
        int acc = 0;
#pragma unroll 1
        for (int k0 = tid * 8; k0 < Kpad; k0 += kStep * kBatch) {
            Raw8<IN_KIND> x[kBatch], sc[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int k8 = k0 + u * kStep;
                x[u].a = x[u].b = make_uint4(0u, 0u, 0u, 0u);     // columns K..Kpad quantise to zero
                sc[u].a = sc[u].b = make_uint4(0u, 0u, 0u, 0u);
                if (k8 < K) {
                    load_raw<IN_KIND>(jb.in, t * jb.ld_in + k8, x[u], tc);
                    if (kHasPre) load_raw<IN_KIND>(jb.pre, k8, sc[u], tc);
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int k8 = k0 + u * kStep;
                if (k8 < Kpad) {
                    const int j = (k8 >> 5) & 7;
                    float v[8], s[8];
                    to_float8<IN_KIND>(x[u], v);
                    if (kHasPre) to_float8<IN_KIND>(sc[u], s);
                    uint32_t Y[8];  // class-shifted operands
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int X = __float2int_rn((kHasPre ? v[e] * s[e] : v[e]) * inv);
                        acc += X;
                        Y[e] = (uint32_t)class_shift(X, j);
                    }
                    store_terms(Y, r0, stride, k8);
                }
            }
        }
        acc = __reduce_add_sync(0xffffffffu, acc);
        if (lane == 0 && acc != 0) atomicAdd(&sumx[t], acc);
    }
    __syncthreads();
}

// Vector path for inputs with at most one 8-column block per thread (T * Kpad / 8 <= threads, e.g. one token of
// 4096 columns): each value is loaded once and stays in registers between the max pass and the conversion, so
// the phase pays a single memory round trip for its input.  Kpad / 8 is a multiple of 32: a warp serves one token.
template <int IN_KIND>
__device__ __noinline__ void quantise_one(const Job& jb, int T, int8_t* xq, int stride, float* red,
                                          int* sumx, float* delta, TagCtx& tc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, nv8 = jb.chunks * 32;
    constexpr bool kHasPre = (IN_KIND != KIND_T);
    const int t = tid / nv8, k8 = (tid - t * nv8) * 8;
    const bool active = t < T;
    float p[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] = 0.f;
    if (!kHasPre) tag_ensure(tc);          // the tagged intermediate is compared with the tag as it is loaded
    Raw8<IN_KIND> xr, sr;
    xr.a = xr.b = sr.a = sr.b = make_uint4(0u, 0u, 0u, 0u);
    if (active && k8 < K) {
        load_raw<IN_KIND>(jb.in, t * jb.ld_in + k8, xr, tc);
        if (kHasPre) load_raw<IN_KIND>(jb.pre, k8, sr, tc);
    }
    if (kHasPre) tag_ensure(tc);           // behind the input loads: the two round trips overlap
    if (active && k8 < K) {
        to_float8<IN_KIND>(xr, p);
        if (kHasPre) {
            float s[8];
            to_float8<IN_KIND>(sr, s);
#pragma unroll
            for (int e = 0; e < 8; ++e) p[e] *= s[e];
        }
    }
    float m = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(p[e]));
    m = warp_max_abs(m);
    // per-warp maxima in the [token][warp] table: a warp contributes to its token only
    if (lane < kMaxTok) red[lane * kGemvWarps + warp] = (active && lane == t) ? m : 0.f;
    if (tid < kMaxTok) sumx[tid] = 0;
    asm volatile("" ::"r"(tc.tag));   // the tag is in this thread's hands before the CTA can arrive at the counter
    __syncthreads();
    if (active) {
        const float inv = token_inv(red, t, k8 == 0, delta);
        const int j = (k8 >> 5) & 7;
        uint32_t Y[8];
        int acc = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int X = __float2int_rn(p[e] * inv);
            acc += X;
            Y[e] = (uint32_t)class_shift(X, j);
        }
        store_terms(Y, xq + (3 * t) * stride, stride, k8);
        acc = __reduce_add_sync(0xffffffffu, acc);
        if (lane == 0 && acc != 0) atomicAdd(&sumx[t], acc);
    }
    __syncthreads();
}

// The same with NI (2 or 4) blocks per thread: item f = tid + i * threads covers token f / nv8, columns
// (f % nv8) * 8.  All NI loads of a thread are in flight together (the tagged intermediate is polled item by
// item, but its later items are valid by then), nothing is loaded twice, and several tokens cost one memory
// round trip instead of one per token and pass.
template <int IN_KIND, int NI>
__device__ __noinline__ void quantise_few(const Job& jb, int T, int8_t* xq, int stride, float* red,
                                          int* sumx, float* delta, TagCtx& tc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, nv8 = jb.chunks * 32, items = T * nv8;
    constexpr bool kHasPre = (IN_KIND != KIND_T);
    float p[NI][8];
    int tt[NI], kk[NI];
    Raw8<IN_KIND> x[NI], sc[NI];
    if (!kHasPre) tag_ensure(tc);
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int f = tid + i * kGemvThreads;
        const int t = f / nv8;
        tt[i] = f < items ? t : -1;
        kk[i] = (f - t * nv8) * 8;
        x[i].a = x[i].b = make_uint4(0u, 0u, 0u, 0u);
        sc[i].a = sc[i].b = make_uint4(0u, 0u, 0u, 0u);
        if (tt[i] >= 0 && kk[i] < K) {
            load_raw<IN_KIND>(jb.in, t * jb.ld_in + kk[i], x[i], tc);
            if (kHasPre) load_raw<IN_KIND>(jb.pre, kk[i], sc[i], tc);
        }
    }
    if (kHasPre) tag_ensure(tc);           // behind the input loads: the two round trips overlap
    float wm[kMaxTok];   // this warp's maximum per token (a warp's item belongs to one token)
#pragma unroll
    for (int q = 0; q < kMaxTok; ++q) wm[q] = 0.f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        float s[8], m = 0.f;
        to_float8<IN_KIND>(x[i], p[i]);
        if (kHasPre) {
            to_float8<IN_KIND>(sc[i], s);
#pragma unroll
            for (int e = 0; e < 8; ++e) p[i][e] *= s[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(p[i][e]));
        m = warp_max_abs(m);
#pragma unroll
        for (int q = 0; q < kMaxTok; ++q) wm[q] = tt[i] == q ? fmaxf(wm[q], m) : wm[q];
    }
    if (lane < kMaxTok) {
        float v = wm[0];
#pragma unroll
        for (int q = 1; q < kMaxTok; ++q) v = lane == q ? wm[q] : v;
        red[lane * kGemvWarps + warp] = v;
    }
    if (tid < kMaxTok) sumx[tid] = 0;
    asm volatile("" ::"r"(tc.tag));   // the tag is in this thread's hands before the CTA can arrive at the counter
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        if (tt[i] >= 0) {      // warp-uniform
            const float inv = token_inv(red, tt[i], kk[i] == 0, delta);
            const int j = (kk[i] >> 5) & 7;
            uint32_t Y[8];
            int acc = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int X = __float2int_rn(p[i][e] * inv);
                acc += X;
                Y[e] = (uint32_t)class_shift(X, j);
            }
            store_terms(Y, xq + (3 * tt[i]) * stride, stride, kk[i]);
            acc = __reduce_add_sync(0xffffffffu, acc);
            if (lane == 0 && acc != 0) atomicAdd(&sumx[tt[i]], acc);
        }
    }
    __syncthreads();
}

// Scalar path for unaligned or ragged inputs (any K, any alignment).
__device__ __noinline__ void quantise_scalar(const Job& jb, int T, int scale_kind, int8_t* xq, int stride,
                                             float* red, int* sumx, float* delta, TagCtx& tc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, Kpad = jb.chunks * 256;
    tag_ensure(tc);
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        float m = 0.f;
        for (int k = tid; k < K; k += kGemvThreads) {
            const float s = jb.pre ? load_as_float(jb.pre, k, scale_kind) : 1.f;
            m = fmaxf(m, fabsf((jb.in_kind == KIND_T ? load1_tagged(jb.in, t * jb.ld_in + k, tc) : load_as_float(jb.in, t * jb.ld_in + k, jb.in_kind)) * s));
        }
        m = warp_max_abs(m);
        if (lane == 0) red[t * kGemvWarps + warp] = m;
    }
    if (tid < kMaxTok) sumx[tid] = 0;
    asm volatile("" ::"r"(tc.tag));   // the tag is in this thread's hands before the CTA can arrive at the counter
    __syncthreads();
#pragma unroll 1
    for (int t = 0; t < T; ++t) {
        const float inv = token_inv(red, t, tid == 0, delta);
        int acc = 0;
        for (int k = tid; k < Kpad; k += kGemvThreads) {
            int X = 0;
            if (k < K) {
                const float s = jb.pre ? load_as_float(jb.pre, k, scale_kind) : 1.f;
                X = __float2int_rn((jb.in_kind == KIND_T ? load1_tagged(jb.in, t * jb.ld_in + k, tc) : load_as_float(jb.in, t * jb.ld_in + k, jb.in_kind)) * s * inv);
            }
            acc += X;
            const int y = class_shift(X, (k >> 5) & 7);
            const int pos = xq_pos(k);
            xq[(3 * t) * stride + pos] = (int8_t)(y & 0xFF);
            xq[(3 * t + 1) * stride + pos] = (int8_t)(((y + 0x80) >> 8) & 0xFF);
            xq[(3 * t + 2) * stride + pos] = (int8_t)(((y + 0x8080) >> 16) & 0xFF);
        }
        acc = __reduce_add_sync(0xffffffffu, acc);
        if (lane == 0 && acc != 0) atomicAdd(&sumx[t], acc);
    }
    __syncthreads();
}

__device__ __forceinline__ void quantise_input(const Job& jb, int T, int scale_kind, int8_t* xq, int stride,
                                               float* red, int* sumx, float* delta, TagCtx& tc) {
    if (!jb.vec) quantise_scalar(jb, T, scale_kind, xq, stride, red, sumx, delta, tc);
    else if (T * jb.chunks * 32 <= kGemvThreads) {
        if (jb.in_kind == KIND_T) quantise_one<KIND_T>(jb, T, xq, stride, red, sumx, delta, tc);
        else if (jb.in_kind == KIND_F16) quantise_one<KIND_F16>(jb, T, xq, stride, red, sumx, delta, tc);
        else quantise_one<KIND_BF16>(jb, T, xq, stride, red, sumx, delta, tc);
    }
    else if (T * jb.chunks * 32 <= 2 * kGemvThreads) {
        if (jb.in_kind == KIND_T) quantise_few<KIND_T, 2>(jb, T, xq, stride, red, sumx, delta, tc);
        else if (jb.in_kind == KIND_F16) quantise_few<KIND_F16, 2>(jb, T, xq, stride, red, sumx, delta, tc);
        else quantise_few<KIND_BF16, 2>(jb, T, xq, stride, red, sumx, delta, tc);
    }
    else if (T > 1 && T * jb.chunks * 32 <= 4 * kGemvThreads) {   // one token of that width: quantise_vec measured faster
        if (jb.in_kind == KIND_T) quantise_few<KIND_T, 4>(jb, T, xq, stride, red, sumx, delta, tc);
        else if (jb.in_kind == KIND_F16) quantise_few<KIND_F16, 4>(jb, T, xq, stride, red, sumx, delta, tc);
        else quantise_few<KIND_BF16, 4>(jb, T, xq, stride, red, sumx, delta, tc);
    }
    else if (jb.in_kind == KIND_T) quantise_vec<KIND_T>(jb, T, xq, stride, red, sumx, delta, tc);
    else if (jb.in_kind == KIND_F16) quantise_vec<KIND_F16>(jb, T, xq, stride, red, sumx, delta, tc);
    else quantise_vec<KIND_BF16>(jb, T, xq, stride, red, sumx, delta, tc);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Per-warp cursor over the (tile, chunk) pairs of one job: 1 KB of packed weights per
// pair (two row groups x 256 columns), pairs tile-major, one contiguous range per warp.
struct PairStream {
    int my_items;   // row tiles (32 rows) of this CTA in the job
    int first;      // the first of them (they are consecutive)
    int my_pairs;   // pairs of this warp
    int begin_il, begin_c;   // first pair of this warp: local tile index, chunk
    int l_il, l_c, l_n;      // next pair to fetch
    int slot;                // which half of the output-scale staging buffer this job uses
};

// Every job of a phase has a contiguous range of CTAs of its own, sized by the host in proportion to its
// packed bytes, and a CTA of the range owns a contiguous run of the job's row tiles (32 rows).  A CTA therefore
// prepares the input of exactly one job per phase: a CTA with rows of two jobs would quantise two inputs one
// after the other, a tail of 1.6-2 us that every other CTA waits for in the next phase or launch.
// Returns the CTA's tiles of `jb`: first tile, count.
__device__ __forceinline__ int my_tiles(const Job& jb, int& first) {
    const int b = (int)blockIdx.x - jb.cta0;
    first = 0;
    if (b < 0 || b >= jb.ncta) return 0;
    first = b * jb.t_q + min(b, jb.t_r);
    return jb.t_q + (b < jb.t_r ? 1 : 0);
}

// The constants of a job that the weight stream needs, held in registers: a read of the shared-memory
// descriptor behind an `asm volatile` with a memory clobber would be re-issued in every iteration.
struct StreamJob {
    const uint4* tiles;
    int row_groups, chunks;
};
__device__ __forceinline__ StreamJob stream_job(const Job& jb) {
    StreamJob sj;
    sj.tiles = jb.tiles;
    sj.row_groups = (jb.rows + 15) >> 4;
    sj.chunks = jb.chunks;
    return sj;
}

__device__ __forceinline__ void stream_issue(PairStream& st, const StreamJob& sj, uint4* ring, int lane) {
    if (st.l_n < st.my_pairs) {
        const int rg = 2 * (st.first + st.l_il);
        const int rgb = (rg + 1 < sj.row_groups) ? rg + 1 : rg;  // odd tail: re-read, result discarded
        uint4* dst = ring + (st.l_n % kStages) * 64 + lane;
        cp_async16(dst, sj.tiles + ((size_t)rg * sj.chunks + st.l_c) * 32 + lane);
        cp_async16(dst + 32, sj.tiles + ((size_t)rgb * sj.chunks + st.l_c) * 32 + lane);
        if (++st.l_c == sj.chunks) { st.l_c = 0; ++st.l_il; }
        ++st.l_n;
    }
    cp_async_commit();  // always commit so that group counting stays uniform
}

// Set the cursor up and start the first weight loads of a job.  They do not depend on
// the job's input vector, so this runs before the input is ready (for a phase-2 job:
// before the wait for the tagged intermediate, which then overlaps with the loads).
__device__ __forceinline__ void stream_begin(PairStream& st, const Job& jb, uint4* ring, int warp,
                                             int lane, uint16_t* post_s, int max_items) {
    st.my_items = my_tiles(jb, st.first);
    const int npairs = st.my_items * jb.chunks;            // < 2^27: the products below fit 32 bits
    const int p_begin = npairs * warp / kGemvWarps;
    st.my_pairs = npairs * (warp + 1) / kGemvWarps - p_begin;
    st.begin_il = 0;
    st.begin_c = p_begin;
    while (st.begin_c >= jb.chunks) { st.begin_c -= jb.chunks; ++st.begin_il; }   // at most my_items steps
    st.l_il = st.begin_il; st.l_c = st.begin_c; st.l_n = 0;
    st.slot ^= 1;
    // The output scales of this CTA's rows are needed right after the main loop: copy them into shared
    // memory now (part of this thread's first copy group, complete when the main loop has drained).
    if (jb.post_vec) {
        const int row0 = 32 * st.first;
        const int nrows = min(32 * st.my_items, jb.rows - row0);
        const int i = (int)threadIdx.x;
        if (8 * i < nrows)
            cp_async16(post_s + st.slot * (32 * max_items) + 8 * i,
                       static_cast<const uint16_t*>(jb.post) + row0 + 8 * i);
    }
    const StreamJob sj = stream_job(jb);
#pragma unroll
    for (int d = 0; d < kStages - 1; ++d) stream_issue(st, sj, ring, lane);
}

__device__ __forceinline__ bool cta_has_items(const Job& jb) {
    int f;
    return my_tiles(jb, f) > 0;
}

// The whole launch for one CTA: the jobs of phase 1, then the jobs of phase 2 (which poll the
// tagged intermediate).  CG = column groups of 8 MMA columns (3 columns per token).
template <int CG>
__device__ __forceinline__ bool run_all(const Phase* phases, const GemvParams& P, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    constexpr int kCols = 8 * CG;
    // shared memory carve-up
    float* red = reinterpret_cast<float*>(smem);                          // [warps][4] + [4]
    int* sumx = reinterpret_cast<int*>(smem + kRedBytes);                 // [4]
    float* delta = reinterpret_cast<float*>(smem + kRedBytes + 16);       // [4]
    uint4* ring = reinterpret_cast<uint4*>(smem + kFixedBytes) + warp * (kStages * 64);  // [stage][2][32]
    int* s1 = reinterpret_cast<int*>(smem + kFixedBytes + kRingBytes);    // [max_items][32 rows][kCols]
    int8_t* xq = reinterpret_cast<int8_t*>(smem + kFixedBytes + kRingBytes + (size_t)P.max_items * (128 * kCols));
    // output scales of the current and the next job: [2][max_items][32] two-byte entries behind the int8 vectors
    uint16_t* post_s = reinterpret_cast<uint16_t*>(xq + (size_t)3 * P.T * P.xq_stride);

    const int njobs = phases[0].njobs;        // same count in both phases
    auto job_of = [&](int s) -> const Job& { return phases[s >= njobs].job[s >= njobs ? s - njobs : s]; };
    auto next_step = [&](int s) {             // first step >= s in which this CTA owns row tiles
        while (s < 2 * njobs && !cta_has_items(job_of(s))) ++s;
        return s;
    };
    PairStream st;
    st.slot = 0;
    int s = next_step(0);
    if (s < 2 * njobs) {
        const Job& j0 = job_of(s);
        stream_begin(st, j0, ring, warp, lane, post_s, P.max_items);
    }
    // Programmatic dependent launch: everything above (descriptor copy, first weight loads) may overlap
    // with the tail of the previous kernel in the stream; the activations and the scratch (shared with
    // that kernel) are only touched after it has completed.  No-ops without the launch attribute.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // All CTAs of this cooperative grid are resident, so CTAs of the next kernel that start early cannot keep one
    // of ours from being scheduled: let the next kernel begin its prologue wherever an SM frees up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // tag of this launch for the intermediate's {value, tag} pairs (and this CTA's arrival, which nobody waits for)
    TagCtx tc;
    tc.tag = 0u; tc.limit = P.spin_limit; tc.status = P.header + 2; tc.begun = 0u;   // read behind the first input loads
    bool arrived = false;
#pragma unroll 1
    while (true) {
        if (s >= 2 * njobs) break;
        const Job& jb = job_of(s);
        const int chunks = jb.chunks;
        for (int i = tid; i < st.my_items * (32 * kCols); i += kGemvThreads) s1[i] = 0;
        quantise_input(jb, P.T, P.scale_kind, xq, P.xq_stride, red, sumx, delta, tc);
        if (!arrived) {   // behind the CTA barriers of the quantiser
            if (tid == 0) launch_arrive(reinterpret_cast<unsigned long long*>(P.header), blockIdx.x == 0, gridDim.x);
            arrived = true;
        }

        // MMA column n = 8*cg + g reads int8 vector n (= 3*tok + term); unused columns re-read a valid one
        const int8_t* bbase[CG];
#pragma unroll
        for (int cg = 0; cg < CG; ++cg) {
            const int n = 8 * cg + g;
            bbase[cg] = xq + (n < 3 * P.T ? n : 3 * P.T - 1) * P.xq_stride + 8 * q;
        }
        int accA[CG][4], accB[CG][4];
#pragma unroll
        for (int cg = 0; cg < CG; ++cg)
#pragma unroll
            for (int i = 0; i < 4; ++i) { accA[cg][i] = 0; accB[cg][i] = 0; }
        int c_il = st.begin_il, c_c = st.begin_c;
        const StreamJob sj = stream_job(jb);
        const int my_pairs = st.my_pairs;
#pragma unroll 1
        for (int n = 0; n < my_pairs; ++n) {
            stream_issue(st, sj, ring, lane);
            cp_async_wait<kStages - 1>();
            __syncwarp();
            const uint4* slot = ring + (n % kStages) * 64 + lane;
            const uint4 ta = slot[0], tb = slot[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t m = 0x01010101u << j;
#pragma unroll
                for (int cg = 0; cg < CG; ++cg) {
                    const uint2 b = *reinterpret_cast<const uint2*>(bbase[cg] + c_c * 256 + 32 * j);
                    mma_s8(accA[cg], ta.x & m, ta.y & m, ta.z & m, ta.w & m, b.x, b.y);
                    mma_s8(accB[cg], tb.x & m, tb.y & m, tb.z & m, tb.w & m, b.x, b.y);
                }
            }
            __syncwarp();  // every lane has read the slot before it is refilled
            // when this warp leaves the row tile, fold its partial sums into shared memory:
            // lane (g, q) holds rows g / g+8 of both row groups, columns 2q, 2q+1 of each column group
            if (++c_c == chunks || n + 1 == my_pairs) {
                int* dst = s1 + c_il * (32 * kCols);
#pragma unroll
                for (int cg = 0; cg < CG; ++cg) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int col = 8 * cg + 2 * q + (i & 1);
                        const int ra = g + 8 * (i >> 1);
                        if (accA[cg][i] != 0) atomicAdd(&dst[ra * kCols + col], accA[cg][i]);
                        if (accB[cg][i] != 0) atomicAdd(&dst[(16 + ra) * kCols + col], accB[cg][i]);
                        accA[cg][i] = 0;
                        accB[cg][i] = 0;
                    }
                }
                if (c_c == chunks) { c_c = 0; ++c_il; }
            }
        }
        cp_async_wait<0>();
        __syncthreads();
        const int my_items = st.my_items;
        const int first_tile_of_job = st.first;
        const uint16_t* my_post = post_s + st.slot * (32 * P.max_items);
        // finalise: thread -> (token slot, row slot); tokens beyond the slot count and rows beyond the 128 row
        // slots are covered by the strides.  The three column sums of a token are the byte terms of
        // 128 * sum_{bit=1}(X); result = sum(X) - 2 * sum_{bit=1}(X) = sum(X) - terms / 64 (terms is a multiple of 128).
        for (int tok = tid >> 7; tok < P.T; tok += kGemvThreads >> 7) {
            const long long sx = sumx[tok];
            const float dl = delta[tok];
            for (int idx = tid & 127; idx < my_items * 32; idx += 128) {
                const int row = 32 * first_tile_of_job + idx;
                if (row < jb.rows) {
                    float extra = 0.f;       // bias and residual of this output (phase 2), fetched before the arithmetic
                    if (jb.bias) extra = load_as_float(jb.bias, row, P.scale_kind);
                    if (jb.resid) extra += load_as_float(jb.resid, tok * jb.ld_res + row, P.scale_kind);
                    const int* c = s1 + idx * kCols + 3 * tok;
                    const long long terms = (long long)c[2] * 65536 + (long long)c[1] * 256 + (long long)c[0];
                    float val = (float)(sx - (terms >> 6)) * dl;
                    if (jb.post) val *= jb.post_vec ? load_as_float(my_post, idx, P.scale_kind)
                                                    : load_as_float(jb.post, row, P.scale_kind);
                    if (jb.out_kind == KIND_T) {
                        store_tagged(jb.out, tok * jb.ld_out + row, val, tc.tag);
                    } else if (jb.out_kind == KIND_F16) {
                        // bias and residual in fp32 behind the output scale; same saturation bounds as the reference epilogue
                        val = fminf(fmaxf(val + extra, -64504.0f), 64504.0f);
                        static_cast<__half*>(jb.out)[tok * jb.ld_out + row] = __float2half(val);
                    } else {
                        val = fminf(fmaxf(val + extra, -3.3895313892515355e+38f), 3.3895313892515355e+38f);
                        static_cast<__nv_bfloat16*>(jb.out)[tok * jb.ld_out + row] = __float2bfloat16(val);
                    }
                }
            }
        }
        // Start the next job's weight stream after this job's results are on their way (their stores then
        // overlap the address arithmetic below) and before any barrier, whose wait the loads overlap.
        const int s_next = next_step(s + 1);
        if (s_next < 2 * njobs)
            stream_begin(st, job_of(s_next), ring, warp, lane, post_s, P.max_items);
        __syncthreads();  // xq / s1 are reused by the next job
        s = s_next;
    }
    if (!arrived) {   // a CTA without row tiles in either phase still counts towards the launch
        tag_ensure(tc);
        asm volatile("" ::"r"(tc.tag));
        __syncthreads();
        if (tid == 0) launch_arrive(reinterpret_cast<unsigned long long*>(P.header), blockIdx.x == 0, gridDim.x);
    }
    return true;
}

template <int CG>
__global__ void __launch_bounds__(kGemvThreads, NQ_GEMV_MIN_CTAS) gemv_group_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(16) unsigned char smem[];
    // The descriptors are read with runtime indices; one cooperative copy out of the
    // parameter bank into shared memory replaces many serial constant-cache misses.
    __shared__ __align__(16) Phase sphase[2];
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&P.phase[0]);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&sphase[0]);
        for (int i = threadIdx.x; i < (int)(sizeof(Phase) * 2 / 4); i += kGemvThreads) dst[i] = src[i];
        __syncthreads();
    }
    run_all<CG>(sphase, P, smem);
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

static unsigned g_spin_limit = kSpinLimit;   // polls before a wait for the tagged intermediate gives up

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
    // Number of CTAs: the dependent chain of a launch (broadcast of the input, hand-over of the intermediate,
    // barriers, completion) costs about 15 ns per participating CTA, the stream gains from every SM.  Small
    // launches therefore run on fewer CTAs than there are SMs (measured optimum on 148 SMs: 80-96 CTAs up to
    // 5 MB of packed factors, 128 around 10 MB, all of them from 20 MB), which also lets the next kernel's CTAs
    // start their prologue on the idle SMs.
    const int sms = sm_count();
    size_t packed = 0;
    for (int i = 0; i < n_linears; ++i) packed += (size_t)d[i].R * ((size_t)d[i].N + d[i].M) / 8;
    int grid = packed < (size_t)(3 << 20) ? sms * 3 / 5 : packed < (size_t)(7 << 20) ? sms * 13 / 20
               : packed < (size_t)(20 << 20) ? sms * 7 / 8 : sms;
    if (grid < kMaxJobs) grid = sms;
    int cta_n[2][kMaxJobs];
    int max_items = 1;
    for (int ph = 0; ph < 2; ++ph) {
        // deal the CTAs to the jobs of the phase: every job gets a contiguous range, sized so that the longest
        // per-CTA stream (row tiles x chunks) is as short as possible
        int items[kMaxJobs], chunks[kMaxJobs];
        for (int i = 0; i < n_linears; ++i) {
            items[i] = ((ph ? d[i].M : d[i].R) + 31) / 32;
            chunks[i] = ((ph ? d[i].R : d[i].N) + 255) / 256;
            cta_n[ph][i] = 1;
        }
        for (int used = n_linears; used < grid; ++used) {
            int best = -1;
            long long best_cost = -1;
            for (int i = 0; i < n_linears; ++i) {
                if (cta_n[ph][i] >= items[i]) continue;      // one tile per CTA already
                const long long cost = (long long)((items[i] + cta_n[ph][i] - 1) / cta_n[ph][i]) * chunks[i];
                if (cost > best_cost) { best_cost = cost; best = i; }
            }
            if (best < 0) break;
            ++cta_n[ph][best];
        }
        for (int i = 0; i < n_linears; ++i) {
            const int most = (items[i] + cta_n[ph][i] - 1) / cta_n[ph][i];
            max_items = most > max_items ? most : max_items;
        }
    }
    const int kpad = (maxK + 255) / 256 * 256;
    const int stride = kpad + 32;  // 32 mod 128: conflict-free 64-bit fragment loads

    // tokens are processed in groups that fit the MMA columns (3 per token) and shared memory
    auto cg_for = [](int t) { return t <= 2 ? 1 : 2; };
    auto smem_for = [&](int t) {
        return kFixedBytes + kRingBytes + (size_t)max_items * (128 * 8 * cg_for(t)) + (size_t)3 * t * stride +
               (size_t)max_items * 128;   // + output scales of two jobs
    };
    int tg = T < kMaxTok ? T : kMaxTok;
    while (tg > 1 && smem_for(tg) > (size_t)smem_limit) --tg;
    if (smem_for(tg) > (size_t)smem_limit) return NQ_ERR_UNSUPPORTED;

    const size_t esz = 2;
    for (int t0 = 0; t0 < T; t0 += tg) {
        const int tn = (T - t0) < tg ? (T - t0) : tg;
        GemvParams P;
        memset(&P, 0, sizeof(P));
        P.header = static_cast<unsigned*>(scratch);
        P.spin_limit = g_spin_limit;
        P.T = tn;
        P.scale_kind = dtype;
        P.xq_stride = stride;
        P.max_items = max_items;
        P.phase[0].njobs = P.phase[1].njobs = n_linears;
        size_t off = kHeaderBytes;
        int cta_a = 0, cta_b = 0;       // first CTA of the next job's range in the two phases
        for (int i = 0; i < n_linears; ++i) {
            const nq_linear_desc& L = d[i];
            void* tbuf = static_cast<char*>(scratch) + off;   // {fp32, tag} pairs, 8 bytes per element
            off += round_up((size_t)kMaxTok * (size_t)L.R * sizeof(uint2), 256);
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
            a.out_kind = KIND_T;
            a.vec = (L.N % 8 == 0) && (L.ldx % 8 == 0) && aligned16(a.in) && aligned16(L.s_in);
            a.post_vec = L.s_mid && (L.R % 8 == 0) && aligned16(L.s_mid);
            a.cta0 = cta_a;
            a.ncta = cta_n[0][i];
            a.t_q = a.items / a.ncta;
            a.t_r = a.items % a.ncta;
            cta_a += a.ncta;
            Job& b = P.phase[1].job[i];
            b.tiles = static_cast<const uint4*>(L.u_tiles);
            b.in = tbuf;
            b.pre = nullptr;
            b.post = L.s_out;
            b.out = static_cast<char*>(L.y) + (size_t)t0 * L.ldy * esz;
            b.bias = L.bias;
            b.resid = L.residual ? static_cast<const char*>(L.residual) + (size_t)t0 * L.ldr * esz : nullptr;
            b.ld_res = L.ldr;
            b.ld_in = L.R;
            b.ld_out = L.ldy;
            b.rows = L.M;
            b.K = L.R;
            b.chunks = (L.R + 255) / 256;
            b.items = (L.M + 31) / 32;
            b.in_kind = KIND_T;
            b.out_kind = dtype;
            b.vec = (L.R % 8 == 0);  // the intermediate lives in the 256-byte aligned scratch
            b.post_vec = (L.M % 8 == 0) && aligned16(L.s_out);
            b.cta0 = cta_b;
            b.ncta = cta_n[1][i];
            b.t_q = b.items / b.ncta;
            b.t_r = b.items % b.ncta;
            cta_b += b.ncta;
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
