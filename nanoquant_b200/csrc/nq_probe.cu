// Measurement probes: small synthetic kernels that isolate one cost of the decode GEMV, timed inside the call.
// They exist so that the figures the design rests on can be re-measured from the repository
// (`python bench.py --mode probe`); nothing on the hot path calls them.
//
//   nq_probe_chain   the dependent chain of one decode launch with the arithmetic taken out: dependency wait,
//                    broadcast load of the input by every CTA, CTA barrier, tagged hand-over of a rank-R vector
//                    between all CTAs, barriers, output store; cooperative launches with programmatic stream
//                    serialization replayed from a CUDA graph, like the real kernel.  Its time per launch is the
//                    floor of the launch structure for a given number of CTAs.
//   nq_probe_loop    the item loop of the GEMV (64 LOP3 + 16 integer MMAs per KB of packed factors) fed in three
//                    ways: from shared memory only (the arithmetic ceiling), through a cp.async ring, and through
//                    registers (streaming loads, four items ahead).
#include <cstdio>

#include "nq_common.cuh"

namespace nq {

struct ChainParams {
    const uint4* x;
    unsigned long long* t;
    uint4* y;
    unsigned long long* counter;
    int n_x16, R, pause_ns;
};

__global__ void __launch_bounds__(512, 1) probe_chain_kernel(const __grid_constant__ ChainParams p) {
    __shared__ float red[16];
    const int tid = threadIdx.x, b = blockIdx.x, G = gridDim.x;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tid < p.n_x16) v = p.x[tid];                       // every CTA reads all of the input
    unsigned long long c;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(p.counter) : "memory");
    const unsigned tag = 0x7FF00000u | ((unsigned)(c / kTagSpan) & 0xFFFFFu);
    float m = __uint_as_float(v.x) + __uint_as_float(v.y) + __uint_as_float(v.z) + __uint_as_float(v.w);
    for (int o = 16; o; o >>= 1) m += __shfl_xor_sync(0xffffffffu, m, o);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    asm volatile("" ::"r"(tag));
    __syncthreads();
    if (tid == 0) launch_arrive(p.counter, b == 0, G);
    float s = 0.f;
    for (int i = 0; i < 16; ++i) s += red[i];
    const int per = (p.R + G - 1) / G;                     // this CTA's slice of the intermediate, tagged
    if (tid < per && b * per + tid < p.R) store_tagged(p.t, b * per + tid, s + tid, tag);
    if (p.pause_ns) __nanosleep(p.pause_ns);
    float acc = 0.f;
    for (int i = tid * 2; i < p.R; i += 1024) {            // every CTA polls all of it
        unsigned long long e0, e1;
        for (unsigned spins = 0; spins < kSpinLimit; ++spins) {
            asm volatile("ld.relaxed.gpu.global.v2.b64 {%0,%1}, [%2];" : "=l"(e0), "=l"(e1) : "l"(p.t + i) : "memory");
            if ((unsigned)(e0 >> 32) == tag && (unsigned)(e1 >> 32) == tag) break;
        }
        acc += __uint_as_float((unsigned)e0) + __uint_as_float((unsigned)e1);
    }
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = acc;
    __syncthreads();
    if (tid < 4) {
        float r = 0;
        for (int i = 0; i < 16; ++i) r += red[i];
        p.y[b * 4 + tid] = make_uint4(__float_as_uint(r), tid, b, 0);
    }
}

__device__ __forceinline__ void probe_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MODE 0: tiles already in shared memory; 1: cp.async ring of four 1 KB slots per warp; 2: registers, four items ahead
template <int MODE>
__global__ void __launch_bounds__(512, 1) probe_loop_kernel(const uint4* w, int* out, int items) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < (65536 + 8192) / 4; i += 512) reinterpret_cast<int*>(smem)[i] = i * 2654435761u;
    __syncthreads();
    const unsigned char* ring_rd = smem + warp * 4096 + lane * 16;
    const unsigned ring_lane = (unsigned)__cvta_generic_to_shared(smem) + warp * 4096u + lane * 16u;
    const int8_t* bbase = reinterpret_cast<const int8_t*>(smem + 65536) + (lane >> 2) * 1024 + 8 * (lane & 3);
    const uint4* next = w + ((size_t)(blockIdx.x * 16 + warp) * items) * 64 + lane;
    int acc[2][2][4] = {};
    int boff = 0;
    auto item = [&](const uint4& ta, const uint4& tb) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t m = 0x01010101u << j;
            const uint2 b = *reinterpret_cast<const uint2*>(bbase + boff + 32 * j);
            probe_mma(acc[0][j & 1], ta.x & m, ta.y & m, ta.z & m, ta.w & m, b.x, b.y);
            probe_mma(acc[1][j & 1], tb.x & m, tb.y & m, tb.z & m, tb.w & m, b.x, b.y);
        }
        boff = (boff + 256) & 767;
    };
    if (MODE == 0) {
        unsigned slot = 0;
#pragma unroll 1
        for (int n = items; n > 0; --n) {
            item(*reinterpret_cast<const uint4*>(ring_rd + slot), *reinterpret_cast<const uint4*>(ring_rd + slot + 512));
            slot = (slot + 1024u) & 4095u;
        }
    } else if (MODE == 1) {
        int n_left = items;
        unsigned f_slot = 0, slot = 0;
        auto issue = [&]() {
            if (n_left > 0) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lane + f_slot), "l"(next) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_lane + f_slot + 512u), "l"(next + 32) : "memory");
                f_slot = (f_slot + 1024u) & 4095u; next += 64; --n_left;
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        for (int i = 0; i < 3; ++i) issue();
#pragma unroll 1
        for (int n = items; n > 0; --n) {
            issue();
            asm volatile("cp.async.wait_group 3;" ::: "memory");
            item(*reinterpret_cast<const uint4*>(ring_rd + slot), *reinterpret_cast<const uint4*>(ring_rd + slot + 512));
            slot = (slot + 1024u) & 4095u;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        uint4 ra[4], rb[4];
#pragma unroll
        for (int d = 0; d < 4; ++d) { ra[d] = __ldcs(next); rb[d] = __ldcs(next + 32); next += 64; }
#pragma unroll 1
        for (int n = items; n > 0; n -= 4) {
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const uint4 ta = ra[d], tb = rb[d];
                if (n > 4) { ra[d] = __ldcs(next); rb[d] = __ldcs(next + 32); next += 64; }
                item(ta, tb);
            }
        }
    }
    int s = 0;
    for (int a = 0; a < 2; ++a) for (int c = 0; c < 2; ++c) for (int i = 0; i < 4; ++i) s += acc[a][c][i];
    out[blockIdx.x * 512 + tid] = s;
}

}  // namespace nq

using namespace nq;

extern "C" {

int nq_probe_chain(int ctas, int R, int pause_ns, float* us_per_launch_host) {
    if (!us_per_launch_host) return NQ_ERR_NULL;
    if (ctas < 1 || ctas > sm_count() || R < 2 || R > 8192 || (R & 1)) return NQ_ERR_SHAPE;
    const int NX = 512;   // 8 KB of input
    uint4* x = nullptr; unsigned long long* t = nullptr; uint4* y = nullptr; unsigned long long* counter = nullptr;
    NQ_CUDA_TRY(cudaMalloc(&x, NX * 16));
    NQ_CUDA_TRY(cudaMalloc(&t, 8192 * 8));
    NQ_CUDA_TRY(cudaMalloc(&y, (size_t)ctas * 4 * 16));
    NQ_CUDA_TRY(cudaMalloc(&counter, 256));
    NQ_CUDA_TRY(cudaMemset(x, 0, NX * 16));
    NQ_CUDA_TRY(cudaMemset(t, 0, 8192 * 8));
    NQ_CUDA_TRY(cudaMemset(counter, 0, 256));
    cudaStream_t st;
    NQ_CUDA_TRY(cudaStreamCreate(&st));
    ChainParams p{x, t, y, counter, NX, R, pause_ns};
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ge = nullptr;
    int rc = NQ_OK;
    NQ_CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    for (int i = 0; i < 100 && rc == NQ_OK; ++i) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(512); cfg.stream = st;
        cudaLaunchAttribute a[2];
        a[0].id = cudaLaunchAttributeCooperative; a[0].val.cooperative = 1;
        a[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; a[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = a; cfg.numAttrs = 2;
        void* args[] = {&p};
        rc = check_cuda(cudaLaunchKernelExC(&cfg, (const void*)probe_chain_kernel, args), "probe launch");
    }
    cudaError_t e = cudaStreamEndCapture(st, &g);
    if (rc == NQ_OK) rc = check_cuda(e, "end capture");
    if (rc == NQ_OK) rc = check_cuda(cudaGraphInstantiate(&ge, g, 0), "instantiate");
    if (rc == NQ_OK) {
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        cudaGraphLaunch(ge, st);
        cudaStreamSynchronize(st);
        cudaEventRecord(e0, st);
        for (int i = 0; i < 10; ++i) cudaGraphLaunch(ge, st);
        cudaEventRecord(e1, st);
        rc = check_cuda(cudaEventSynchronize(e1), "probe run");
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        *us_per_launch_host = ms * 1e3f / 1000.f;
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    if (ge) cudaGraphExecDestroy(ge);
    if (g) cudaGraphDestroy(g);
    cudaStreamDestroy(st);
    cudaFree(x); cudaFree(t); cudaFree(y); cudaFree(counter);
    return rc;
}

int nq_probe_loop(int mode, int items_per_warp, float* gbs_host) {
    if (!gbs_host) return NQ_ERR_NULL;
    if (mode < 0 || mode > 2 || items_per_warp < 4 || items_per_warp % 4 || items_per_warp > 1024) return NQ_ERR_SHAPE;
    const int ctas = sm_count();
    const size_t bytes = (size_t)ctas * 16 * items_per_warp * 1024;
    uint4* w = nullptr; int* out = nullptr;
    NQ_CUDA_TRY(cudaMalloc(&w, bytes + 65536));
    NQ_CUDA_TRY(cudaMalloc(&out, (size_t)ctas * 512 * 4));
    NQ_CUDA_TRY(cudaMemset(w, 0x5a, bytes));
    const int sm = 65536 + 8192;
    const void* fn = mode == 0 ? (const void*)probe_loop_kernel<0> : mode == 1 ? (const void*)probe_loop_kernel<1>
                                                                               : (const void*)probe_loop_kernel<2>;
    int rc = check_cuda(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, sm), "smem attribute");
    if (rc == NQ_OK) {
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        void* args[] = {&w, &out, &items_per_warp};
        for (int i = 0; i < 2; ++i) cudaLaunchKernel(fn, dim3(ctas), dim3(512), args, sm, 0);
        cudaDeviceSynchronize();
        cudaEventRecord(e0, 0);
        for (int i = 0; i < 5; ++i) cudaLaunchKernel(fn, dim3(ctas), dim3(512), args, sm, 0);
        cudaEventRecord(e1, 0);
        rc = check_cuda(cudaEventSynchronize(e1), "probe run");
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        *gbs_host = (float)((double)bytes * 5 / (ms * 1e-3) / 1e9);
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    cudaFree(w); cudaFree(out);
    return rc;
}

}  // extern "C"
