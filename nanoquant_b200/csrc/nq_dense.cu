// Dense 16-bit GEMV for the un-quantised head of a decode step:
//
//     y[t, v] = sum_k x[t, k] * W[v, k] (+ bias[v])        W [V, N] fp16 / bf16 row-major, 1 <= T <= 16
//
// The reference keeps `lm_head` as a plain nn.Linear in the model dtype (it is not in the list of quantised
// linears), so every decoded token streams V * N * 2 bytes of it (1.24 GB for a 151936 x 4096 head).  The
// kernel is HBM bound: W is read exactly once with 16-byte streaming loads, straight from global memory into
// the A fragments of mma.sync.m16n8k16 (16 weight rows x 8 tokens per instruction, fp32 accumulation); the
// tokens are the MMA's N dimension, so up to 8 of them cost the same instructions as one.
//
// Work split.  A unit is 16 consecutive rows of W.  The 16 (above 8 tokens: 32) warps of a CTA split the K dimension of a unit
// in batches of 4 k blocks (32 columns each) per warp, keep 8 x 16-byte loads per lane in flight, and add
// their partial 16 x 8 accumulators through shared memory (double buffered: one CTA barrier per 16 rows =
// per 128 KB of weights at N = 4096).  CTAs own contiguous, equally sized ranges of units.
//
// Fragment mapping.  Lane (g, q) = (lane / 4, lane % 4) loads the 16 bytes at columns 32*blk + 8q .. 8q+7 of
// rows g and g + 8.  Their four 32-bit registers r0..r3 feed two MMAs: {r0, r1} and {r2, r3} as the
// (k-slot 2q, 2q+8) register pairs; the same lane takes x[token g][32*blk + 8q ..] as one 16-byte shared
// load whose registers are the matching B fragments.  The k slots of an MMA are a permutation of the
// columns, the same for A and B, so the sum is unchanged.
#include "nq_common.cuh"

namespace nq {

// 16 warps per CTA and two CTAs per SM for up to 8 tokens; 32 warps and one CTA per SM above (16 tokens of a
// wide row leave shared memory for one CTA only, and the loads in flight per SM stay the same)
constexpr int kDenseBlocksPerBatch = 4;   // k blocks of 32 columns per warp per batch
constexpr int kDenseMaxTokens = 16;

struct DenseParams {
    const char* w;
    const char* x;
    void* y;
    const void* bias;      // nullable
    long long ldw_bytes;
    long long ldy;         // elements between tokens of y
    int T, N, V;
    int units;             // ceil(V / 16)
    int nbat;              // batches per unit
    int x_stride;          // bytes between tokens in shared memory
};

__device__ __forceinline__ uint4 ldg_stream16(const char* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                     "{%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                     "{%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

template <bool BF16>
__device__ __forceinline__ float load_scalar(const void* p, long long i) {
    if constexpr (BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    else return __half2float(static_cast<const __half*>(p)[i]);
}
template <bool BF16>
__device__ __forceinline__ void store_scalar(void* p, long long i, float v) {
    if constexpr (BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

// NB = token blocks of 8 (1: T <= 8, 2: T <= 16).
template <int NB, bool BF16>
__global__ void __launch_bounds__(512 * NB, 2 / NB) dense_gemv_kernel(const DenseParams P) {
    constexpr int kDenseWarps = 16 * NB, kDenseThreads = 32 * kDenseWarps;
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xs = smem;                                                  // [T][x_stride]
    float* part = reinterpret_cast<float*>(smem + (size_t)P.T * P.x_stride);   // [kBuffers][warps][NB][4][32]
    constexpr int kPartPerWarp = NB * 4 * 32;
    // Shared memory that a CTA holds is taken from the SM's L1, through which the streaming loads in flight pass:
    // with 16 tokens of a wide row resident, a second partial-sum buffer costs more bandwidth than the extra CTA
    // barrier of a single one.
    constexpr int kBuffers = NB == 1 ? 2 : 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;

    // tokens -> shared memory, zero behind column N (the padded k blocks multiply zero weights, which must
    // not meet a NaN)
    {
        const int chunks = P.x_stride / 16;          // 16-byte chunks per token, padding included
        const int valid = P.N / 8, total = P.T * chunks;
        for (int i0 = tid; i0 < total; i0 += 4 * kDenseThreads) {   // four independent loads per round trip
            uint4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * kDenseThreads, t = i / chunks, c = i - t * chunks;
                v[k] = make_uint4(0, 0, 0, 0);
                if (i < total && c < valid) v[k] = ldg_stream16(P.x + ((size_t)t * P.N + (size_t)c * 8) * 2);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * kDenseThreads, t = i / chunks, c = i - t * chunks;
                if (i < total) *reinterpret_cast<uint4*>(xs + (size_t)t * P.x_stride + (size_t)c * 16) = v[k];
            }
        }
    }
    __syncthreads();

    const int u0 = (int)((long long)blockIdx.x * P.units / gridDim.x);
    const int u1 = (int)((long long)(blockIdx.x + 1) * P.units / gridDim.x);
    const bool tok0 = g < P.T, tok1 = NB > 1 && g + 8 < P.T;
    const unsigned char* x0 = xs + (size_t)(tok0 ? g : 0) * P.x_stride + q * 16;
    const unsigned char* x1 = xs + (size_t)(tok1 ? g + 8 : 0) * P.x_stride + q * 16;

    // One batch of weights per lane: 2 rows x 4 k blocks x 16 bytes.  The batch of the NEXT (unit, batch) step is
    // requested right after the MMAs have consumed the registers of the current one, i.e. before the CTA barrier
    // and the reduction that end a unit, so the stream of loads never drains.
    uint4 wa[kDenseBlocksPerBatch], wb[kDenseBlocksPerBatch];
    auto load_batch = [&](int u, int b) {
        const int ra = min(u * 16 + g, P.V - 1), rb = min(u * 16 + g + 8, P.V - 1);   // clamped: never stored
        const int blk0 = (b * kDenseWarps + warp) * kDenseBlocksPerBatch;
        const char* pa = P.w + (long long)ra * P.ldw_bytes + q * 16 + (size_t)blk0 * 64;
        const char* pb = P.w + (long long)rb * P.ldw_bytes + q * 16 + (size_t)blk0 * 64;
#pragma unroll
        for (int j = 0; j < kDenseBlocksPerBatch; ++j) {
            const int k0 = (blk0 + j) * 32 + q * 8;
            if (k0 < P.N) {
                wa[j] = ldg_stream16(pa + j * 64);
                wb[j] = ldg_stream16(pb + j * 64);
            } else {
                wa[j] = make_uint4(0, 0, 0, 0);
                wb[j] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    float acc[NB][4];
#pragma unroll
    for (int n = 0; n < NB; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    if (u0 < u1) load_batch(u0, 0);

    for (int u = u0, b = 0; u < u1;) {
        {
            const int blk0 = (b * kDenseWarps + warp) * kDenseBlocksPerBatch;
#pragma unroll
            for (int j = 0; j < kDenseBlocksPerBatch; ++j) {
                const size_t off = (size_t)(blk0 + j) * 64;
                uint4 xv = *reinterpret_cast<const uint4*>(x0 + off);
                if (!tok0) xv = make_uint4(0, 0, 0, 0);
                mma16816<BF16>(acc[0], wa[j].x, wb[j].x, wa[j].y, wb[j].y, xv.x, xv.y);
                mma16816<BF16>(acc[0], wa[j].z, wb[j].z, wa[j].w, wb[j].w, xv.z, xv.w);
                if constexpr (NB > 1) {
                    uint4 xw = *reinterpret_cast<const uint4*>(x1 + off);
                    if (!tok1) xw = make_uint4(0, 0, 0, 0);
                    mma16816<BF16>(acc[1], wa[j].x, wb[j].x, wa[j].y, wb[j].y, xw.x, xw.y);
                    mma16816<BF16>(acc[1], wa[j].z, wb[j].z, wa[j].w, wb[j].w, xw.z, xw.w);
                }
            }
        }
        const bool unit_done = b + 1 == P.nbat;
        const int nu = unit_done ? u + 1 : u, nbt = unit_done ? 0 : b + 1;
        if (nu < u1) load_batch(nu, nbt);
        if (!unit_done) {
            b = nbt;
            continue;
        }

        // partial accumulators of the warps -> shared memory, then 128 * NB threads add them.  With two buffers the
        // barrier of unit u + 1 orders this unit's reads before the writes of unit u + 2 to the same buffer.
        const int buf = kBuffers == 2 ? ((u - u0) & 1) : 0;
        float* mine = part + ((size_t)buf * kDenseWarps + warp) * kPartPerWarp;
#pragma unroll
        for (int n = 0; n < NB; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) mine[(n * 4 + i) * 32 + lane] = acc[n][i];
        __syncthreads();
        if (tid < 128 * NB) {
            // thread -> (token, row) with the row fastest, so that a token's 16 outputs are one 32-byte run
            const int n = tid >> 4, row = tid & 15;
            const int nb = n >> 3, nn = n & 7;
            // accumulator register i of lane (g', q') is row g' + 8 * (i / 2), token 2 q' + (i % 2)
            const int reg = (row >> 3) * 2 + (nn & 1), src_lane = (row & 7) * 4 + (nn >> 1);
            const float* src = part + (size_t)buf * kDenseWarps * kPartPerWarp + (nb * 4 + reg) * 32 + src_lane;
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kDenseWarps; ++w) s += src[w * kPartPerWarp];
            const int v = u * 16 + row;
            if (n < P.T && v < P.V) {
                if (P.bias) s += load_scalar<BF16>(P.bias, v);
                store_scalar<BF16>(P.y, (long long)n * P.ldy + v, s);
            }
        }
        if constexpr (kBuffers == 1) __syncthreads();   // the sums are read before the next unit overwrites them
#pragma unroll
        for (int n = 0; n < NB; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
        u = nu;
        b = 0;
    }
}

template <int NB, bool BF16>
int launch_dense(const DenseParams& P, size_t smem, int optin, cudaStream_t stream) {
    constexpr int kDenseThreads = 512 * NB;
    static int configured[64] = {0};    // per device: 0 = not yet, else CTAs per SM + 1
    int dev = 0;
    NQ_CUDA_TRY(cudaGetDevice(&dev));
    const void* fn = (const void*)dense_gemv_kernel<NB, BF16>;
    if (!configured[dev & 63]) {
        NQ_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, optin));
        configured[dev & 63] = 1;
    }
    int per_sm = 0;
    NQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kDenseThreads, smem));
    if (per_sm < 1) return NQ_ERR_TOO_LARGE;
    long long grid = (long long)per_sm * sm_count();
    if (grid > P.units) grid = P.units;
    dense_gemv_kernel<NB, BF16><<<(unsigned)grid, kDenseThreads, smem, stream>>>(P);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

}  // namespace nq

using namespace nq;

extern "C" {

int nq_dense_gemv_max_tokens(void) { return kDenseMaxTokens; }

int nq_dense_gemv_fwd(const void* x, const void* w, const void* bias, void* y, int T, int N, int V,
                      int64_t ldw, int64_t ldy, int dtype, nq_stream_t stream) {
    if (!x || !w || !y) return NQ_ERR_NULL;
    if (dtype != NQ_F16 && dtype != NQ_BF16) return NQ_ERR_DTYPE;
    if (T < 1 || N < 1 || V < 1 || N % 8 || ldw < N || ldw % 8 || ldy < V) return NQ_ERR_SHAPE;
    if (T > kDenseMaxTokens) return NQ_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(w)) return NQ_ERR_ALIGN;

    const int nblk = (N + 31) / 32;
    auto warps_for = [](int t) { return t > 8 ? 32 : 16; };
    auto nbat_for = [&](int t) {
        const int per_batch = warps_for(t) * kDenseBlocksPerBatch;
        return (nblk + per_batch - 1) / per_batch;
    };
    // token stride: the padded row plus 64 bytes, so that the eight lanes of a quarter warp (two tokens x four
    // 16-byte chunks) hit eight different 16-byte bank groups
    auto stride_for = [&](int t) { return nbat_for(t) * warps_for(t) * kDenseBlocksPerBatch * 64 + 64; };
    auto smem_for = [&](int t) {
        return (size_t)t * stride_for(t) + (size_t)(t > 8 ? 1 : 2) * warps_for(t) * (t > 8 ? 2 : 1) * 4 * 32 * sizeof(float);
    };
    int dev = 0, optin = 0;
    NQ_CUDA_TRY(cudaGetDevice(&dev));
    NQ_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    // all tokens of a launch sit in shared memory; where they do not fit (wide rows, many tokens) the tokens
    // go in several launches, each streaming w once
    int chunk = T;
    while (chunk > 1 && smem_for(chunk) > (size_t)optin) chunk = (chunk + 1) / 2;
    if (smem_for(chunk) > (size_t)optin) return NQ_ERR_TOO_LARGE;

    cudaStream_t s = as_stream(stream);
    for (int t0 = 0; t0 < T; t0 += chunk) {
        DenseParams P;
        P.T = T - t0 < chunk ? T - t0 : chunk;
        P.w = static_cast<const char*>(w);
        P.x = static_cast<const char*>(x) + (size_t)t0 * N * 2;
        P.y = static_cast<char*>(y) + (size_t)t0 * ldy * 2;
        P.bias = bias;
        P.ldw_bytes = ldw * 2;
        P.ldy = ldy;
        P.N = N;
        P.V = V;
        P.units = (V + 15) / 16;
        P.nbat = nbat_for(P.T);
        P.x_stride = stride_for(P.T);
        const size_t smem = smem_for(P.T);
        int st;
        if (dtype == NQ_BF16) st = P.T > 8 ? launch_dense<2, true>(P, smem, optin, s) : launch_dense<1, true>(P, smem, optin, s);
        else st = P.T > 8 ? launch_dense<2, false>(P, smem, optin, s) : launch_dense<1, false>(P, smem, optin, s);
        if (st != NQ_OK) return st;
    }
    return NQ_OK;
}

}  // extern "C"
