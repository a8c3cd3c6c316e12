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

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kMaxJobs = 4;         // linears per launch
constexpr int kMaxTok = 4;          // tokens per launch (2 int8 terms each -> 8 MMA columns)
constexpr int kQMax = 32639;        // 127*256 + 127: hi and lo both fit a signed byte
constexpr int kPrefetch = 6;        // tile pairs in flight per lane
constexpr unsigned kSpinLimit = 4000000u;
constexpr size_t kHeaderBytes = 256;

enum : int { KIND_F16 = 0, KIND_BF16 = 1, KIND_F32 = 2 };

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
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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

// Bounded device-wide barrier.  Returns false when the wait expired.
__device__ bool grid_barrier(unsigned* header, unsigned nblocks) {
    __shared__ int ok;
    __syncthreads();
    if (threadIdx.x == 0) {
        ok = 1;
        volatile unsigned* gen = header + 1;
        const unsigned my_gen = *gen;
        __threadfence();
        const unsigned old = atomicAdd(header, 1u);
        if (old == nblocks - 1) {
            atomicExch(header, 0u);
            __threadfence();
            atomicAdd(header + 1, 1u);
        } else {
            unsigned spins = 0;
            while (*gen == my_gen) {
                if (++spins > kSpinLimit) {
                    atomicExch(header + 2, (unsigned)(-NQ_ERR_TIMEOUT));
                    ok = 0;
                    break;
                }
            }
        }
        __threadfence();
    }
    __syncthreads();
    return ok != 0;
}

// Quantise the input vectors of a job into shared memory.
//   xq: 2*T int8 vectors (row 2*tok = hi term, 2*tok+1 = lo term), `stride` bytes apart,
//       in the k order the MMA B fragments expect (see below); columns K..Kpad are zero.
//   sumx[tok]: sum of the 16-bit values, delta[tok]: value of one unit.
__device__ void quantise_input(const Job& jb, int T, int scale_kind, int8_t* xq, int stride,
                               float* red, int* sumx, float* delta) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = jb.K, Kpad = jb.chunks * 256;
    // pass 1: per-token max |in * pre|
    float mx[kMaxTok] = {0.f, 0.f, 0.f, 0.f};
    for (int k = tid; k < K; k += kGemvThreads) {
        const float s = jb.pre ? load_as_float(jb.pre, k, scale_kind) : 1.f;
#pragma unroll
        for (int t = 0; t < kMaxTok; ++t)
            if (t < T) mx[t] = fmaxf(mx[t], fabsf(load_as_float(jb.in, t * jb.ld_in + k, jb.in_kind) * s));
    }
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[t] = fmaxf(mx[t], __shfl_xor_sync(0xffffffffu, mx[t], o));
        if (lane == 0) red[warp * kMaxTok + t] = mx[t];
    }
    if (tid < kMaxTok) sumx[tid] = 0;
    __syncthreads();
    float inv[kMaxTok];
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) {
        float m = 0.f;
        for (int w = 0; w < kGemvWarps; ++w) m = fmaxf(m, red[w * kMaxTok + t]);
        // a non-finite or zero maximum quantises everything to zero
        const bool good = (m > 0.f) && (m < 3.0e38f);
        inv[t] = good ? (float)kQMax / m : 0.f;
        if (tid == 0) delta[t] = good ? m / (float)kQMax : 0.f;
    }
    // pass 2: four consecutive k per thread -> one 32-bit word of the hi and of the lo vector.
    // Byte position inside a chunk of 256: 32*j + 8*q + 4*h + b for k = 32*j + 16*h + 4*q + b,
    // so that lane (g, q) fetches its two B registers {k=4q.., k=16+4q..} with one 64-bit load.
    int acc[kMaxTok] = {0, 0, 0, 0};
    for (int k4 = tid * 4; k4 < Kpad; k4 += kGemvThreads * 4) {
        const int kin = k4 & 255, j = kin >> 5, h = (kin >> 4) & 1, q = (kin >> 2) & 3;
        const int pos = (k4 & ~255) + 32 * j + 8 * q + 4 * h;
        float s[4];
#pragma unroll
        for (int b = 0; b < 4; ++b)
            s[b] = (k4 + b < K) ? (jb.pre ? load_as_float(jb.pre, k4 + b, scale_kind) : 1.f) : 0.f;
#pragma unroll
        for (int t = 0; t < kMaxTok; ++t) {
            if (t < T) {
                uint32_t hi = 0, lo = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    int X = 0;
                    if (k4 + b < K) {
                        const float v = load_as_float(jb.in, t * jb.ld_in + k4 + b, jb.in_kind) * s[b];
                        X = __float2int_rn(fminf(fmaxf(v * inv[t], -(float)kQMax), (float)kQMax));
                    }
                    acc[t] += X;
                    const int l = (int)(int8_t)(X & 0xFF);   // signed low byte
                    const int hh = (X - l) >> 8;             // exact, in [-127, 127]
                    lo |= (uint32_t)(l & 0xFF) << (8 * b);
                    hi |= (uint32_t)(hh & 0xFF) << (8 * b);
                }
                *reinterpret_cast<uint32_t*>(xq + (2 * t) * stride + pos) = hi;
                *reinterpret_cast<uint32_t*>(xq + (2 * t + 1) * stride + pos) = lo;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < kMaxTok; ++t) {
        if (t < T) {
            int a = acc[t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0 && a != 0) atomicAdd(&sumx[t], a);
        }
    }
    __syncthreads();
}

struct TilePair {
    uint4 a, b;  // row group 2*item and 2*item + 1
};

// One phase: every CTA walks the jobs; inside a job it owns the row tiles
// blockIdx.x, blockIdx.x + gridDim.x, ... and its warps split the K chunks.
__device__ void run_phase(const Phase& ph, const GemvParams& P, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    // shared memory carve-up
    float* red = reinterpret_cast<float*>(smem);                    // [warps][4]
    int* sumx = reinterpret_cast<int*>(smem + 256);                 // [4]
    float* delta = reinterpret_cast<float*>(smem + 256 + 16);       // [4]
    int* s1 = reinterpret_cast<int*>(smem + 512);                   // [max_items][4][32]
    int8_t* xq = reinterpret_cast<int8_t*>(smem + 512 + (size_t)P.max_items * 512);

    for (int ji = 0; ji < ph.njobs; ++ji) {
        const Job& jb = ph.job[ji];
        const int my_items = ((int)blockIdx.x < jb.items)
                                 ? (jb.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        if (my_items == 0) continue;  // uniform per CTA
        const int chunks = jb.chunks;
        const int row_groups = (jb.rows + 15) >> 4;
        const int npairs = my_items * chunks;
        const int my_pairs = (warp < npairs) ? (npairs - 1 - warp) / kGemvWarps + 1 : 0;

        auto tile_ptr = [&](int p, int second) -> const uint4* {
            const int il = p / chunks, c = p - il * chunks;
            int rg = 2 * ((int)blockIdx.x + il * (int)gridDim.x) + second;
            if (rg >= row_groups) rg = row_groups - 1;  // odd tail: re-read, result discarded
            return jb.tiles + ((size_t)rg * chunks + c) * 32 + lane;
        };
        // issue the first weight loads before the input is prepared: they do not depend on it
        TilePair buf[kPrefetch];
#pragma unroll
        for (int d = 0; d < kPrefetch; ++d) {
            if (d < my_pairs) {
                const int p = warp + d * kGemvWarps;
                buf[d].a = load_tile(tile_ptr(p, 0));
                buf[d].b = load_tile(tile_ptr(p, 1));
            }
        }
        for (int i = tid; i < my_items * 128; i += kGemvThreads) s1[i] = 0;
        quantise_input(jb, P.T, P.scale_kind, xq, P.xq_stride, red, sumx, delta);

        const int brow = (g < 2 * P.T) ? g : (2 * P.T - 1);  // unused MMA columns re-read a valid vector
        const int8_t* bbase = xq + brow * P.xq_stride + 8 * q;

        int accA[8][4], accB[8][4];
        int cur_item = -1;
        auto flush = [&]() {
            if (cur_item < 0) return;
            // d_j = 2^j * sum (j < 7), -128 * sum (j = 7): exact shifts
            int v[4] = {0, 0, 0, 0};  // {rows g, g+8 of group A, rows g, g+8 of group B}
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int sg = (j == 7) ? -1 : 1;
                v[0] += sg * (((accA[j][0] >> j) << 8) + (accA[j][1] >> j));
                v[1] += sg * (((accA[j][2] >> j) << 8) + (accA[j][3] >> j));
                v[2] += sg * (((accB[j][0] >> j) << 8) + (accB[j][1] >> j));
                v[3] += sg * (((accB[j][2] >> j) << 8) + (accB[j][3] >> j));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (v[i] != 0) atomicAdd(&s1[(cur_item * 4 + i) * 32 + lane], v[i]);
        };
        auto consume = [&](const TilePair& tp, int p) {
            const int il = p / chunks, c = p - il * chunks;
            if (il != cur_item) {
                flush();
                cur_item = il;
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) { accA[j][i] = 0; accB[j][i] = 0; }
            }
            const uint2* bp = reinterpret_cast<const uint2*>(bbase + c * 256);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint2 b = bp[j * 4];
                const uint32_t m = 0x01010101u << j;
                mma_s8(accA[j], tp.a.x & m, tp.a.y & m, tp.a.z & m, tp.a.w & m, b.x, b.y);
                mma_s8(accB[j], tp.b.x & m, tp.b.y & m, tp.b.z & m, tp.b.w & m, b.x, b.y);
            }
        };
        for (int base = 0; base < my_pairs; base += kPrefetch) {
#pragma unroll
            for (int d = 0; d < kPrefetch; ++d) {
                const int idx = base + d;
                if (idx < my_pairs) {
                    const TilePair tp = buf[d];
                    if (idx + kPrefetch < my_pairs) {
                        const int pn = warp + (idx + kPrefetch) * kGemvWarps;
                        buf[d].a = load_tile(tile_ptr(pn, 0));
                        buf[d].b = load_tile(tile_ptr(pn, 1));
                    }
                    consume(tp, warp + idx * kGemvWarps);
                }
            }
        }
        flush();
        __syncthreads();
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
    }
}

__global__ void __launch_bounds__(kGemvThreads, 1) gemv_group_kernel(const __grid_constant__ GemvParams P) {
    extern __shared__ __align__(16) unsigned char smem[];
    run_phase(P.phase[0], P, smem);
    if (!grid_barrier(P.header, gridDim.x)) return;
    run_phase(P.phase[1], P, smem);
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
    auto smem_for = [&](int t) { return (size_t)512 + (size_t)max_items * 512 + (size_t)2 * t * stride; };
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

int nq_scratch_status(const void* scratch, nq_stream_t stream) {
    if (!scratch) return NQ_ERR_NULL;
    unsigned h[4] = {0, 0, 0, 0};
    NQ_CUDA_TRY(cudaMemcpyAsync(h, scratch, sizeof(h), cudaMemcpyDeviceToHost, as_stream(stream)));
    NQ_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    return h[2] == 0 ? NQ_OK : -(int)h[2];
}

}  // extern "C"
