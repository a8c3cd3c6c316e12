// Shared helpers of the nanoquant_b200 kernels: status handling, argument
// checks and the bit-order conversions of a 32-column word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nanoquant_b200.h"

namespace nq {

// Records the text of a failed CUDA runtime call for nq_last_cuda_error().
void set_cuda_error(cudaError_t e, const char* where);

inline int check_cuda(cudaError_t e, const char* where) {
    if (e == cudaSuccess) return NQ_OK;
    set_cuda_error(e, where);
    return NQ_ERR_CUDA;
}

#define NQ_CUDA_TRY(expr)                                             \
    do {                                                              \
        int _s = ::nq::check_cuda((expr), #expr);                     \
        if (_s != NQ_OK) return _s;                                   \
    } while (0)

// Launch errors surface through cudaGetLastError right after the <<<>>>.
#define NQ_LAUNCH_CHECK() NQ_CUDA_TRY(cudaGetLastError())

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline cudaStream_t as_stream(nq_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Number of SMs of the current device (cached per device).
int sm_count();

// ---------------------------------------------------------------------------
// launch tags: data that carries its own "ready" flag
// ---------------------------------------------------------------------------
// A producer CTA stores every element of an intermediate as an 8-byte {fp32 value, tag} pair with one 64-bit
// store; a consumer CTA of the same launch loads the pairs it needs and repeats the load until every tag
// equals the tag of this launch.  The first poll after the last producer store has landed already returns
// the data, which takes an arrive / poll / reload sequence (three memory round trips) and any device-wide
// barrier off the critical path.  Consumers spin on other CTAs, so the launch must be cooperative.
//
// The tag is the launch count of the scratch buffer, read from a 64-bit arrival counter in its header:
// every launch advances it by exactly kTagSpan (the first CTA adds kTagSpan - (CTAs - 1), every other CTA
// adds 1, with a reduction nobody waits for), so the bits above the span are the same for every CTA of a
// launch whenever it reads them (fewer than a span's worth of arrivals can precede the read) and differ from
// those of every recent launch.  Reads and arrivals of a launch must come after the previous launch on the
// scratch has completed (behind griddepcontrol.wait).  The tag is 0x7FF in its upper 12 bits (a NaN pattern
// as fp32 and in both halves as fp16 / bf16 pairs, which no kernel that shares the scratch ever stores, and
// never the 0 of a zeroed scratch) and the launch count modulo 2^20 below; an element is rewritten by every
// launch that uses its address, so a stale tag can only match after 2^20 launches in a row that leave it
// alone.  Waits are bounded: on expiry a status word is set and the thread goes on with what it has (the
// host reports the status).
constexpr unsigned kTagSpan = 1024u;        // > CTAs per tagged launch
constexpr unsigned kSpinLimit = 4000000u;   // default number of polls before a wait gives up
struct TagCtx {
    unsigned tag;        // tag of this launch
    unsigned limit;      // polls a wait of this thread may still spend; 0 after an expiry (sticky: one missing
                         // producer costs every thread one limit, not one limit per element it waits for)
    unsigned* status;    // device status word (header word 2)
    unsigned begun;      // tag and status have been read
};
// Reads the launch tag and the status word of the scratch header.  Issue it AFTER the first data loads of the
// kernel: its results are first needed when a tag is compared or stored, so the round trips overlap.  A status
// left by an earlier expiry on this scratch disables spinning altogether (the data of such a launch is void anyway).
__device__ __forceinline__ void tag_begin(TagCtx& tc, unsigned* header, unsigned limit) {
    unsigned long long c;
    unsigned st;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(header) : "memory");
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(st) : "l"(header + 2) : "memory");
    tc.tag = 0x7FF00000u | ((unsigned)(c / kTagSpan) & 0xFFFFFu);
    tc.limit = st ? 0u : limit;
    tc.status = header + 2;
    tc.begun = 1u;
}
__device__ __forceinline__ void tag_wait_expired(TagCtx& tc) {
    atomicExch(tc.status, (unsigned)(-NQ_ERR_TIMEOUT));
    tc.limit = 0u;
}
// This CTA's arrival at the counter.  Issued by one thread, once per launch, after a CTA barrier that every
// thread passes behind its own tag_begin() read: the arrival that completes the span would otherwise show
// the next launch's tag to a thread of the same CTA that reads late.
__device__ __forceinline__ void launch_arrive(unsigned long long* counter, bool first_cta, unsigned n_ctas) {
    const unsigned long long w = first_cta ? (unsigned long long)(kTagSpan - (n_ctas - 1)) : 1ull;
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(counter), "l"(w) : "memory");
}
// One 64-bit scalar store: value and tag become visible together (a vector store of two 32-bit words would be two
// accesses in the memory model).
__device__ __forceinline__ void store_tagged(void* base, long long i, float val, unsigned tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(val);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(static_cast<unsigned long long*>(base) + i), "l"(w) : "memory");
}

// ---------------------------------------------------------------------------
// bit orders of a 32-column word
//   lsb_first: element k              -> bit k
//   half2:     element 2j / element 2j+1 -> bit 15-j / bit 31-j
// ---------------------------------------------------------------------------

// keep the even bits of w, squeezed into the low 16 bits
__host__ __device__ inline uint32_t squeeze_even_bits(uint32_t w) {
    uint32_t x = w & 0x55555555u;
    x = (x | (x >> 1)) & 0x33333333u;
    x = (x | (x >> 2)) & 0x0F0F0F0Fu;
    x = (x | (x >> 4)) & 0x00FF00FFu;
    x = (x | (x >> 8)) & 0x0000FFFFu;
    return x;
}

// spread the low 16 bits of v onto the even bit positions
__host__ __device__ inline uint32_t spread_to_even_bits(uint32_t v) {
    uint32_t x = v & 0x0000FFFFu;
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    x = (x | (x << 1)) & 0x55555555u;
    return x;
}

__host__ __device__ inline uint32_t reverse16(uint32_t v) {
    v = ((v & 0x5555u) << 1) | ((v >> 1) & 0x5555u);
    v = ((v & 0x3333u) << 2) | ((v >> 2) & 0x3333u);
    v = ((v & 0x0F0Fu) << 4) | ((v >> 4) & 0x0F0Fu);
    v = ((v & 0x00FFu) << 8) | ((v >> 8) & 0x00FFu);
    return v & 0xFFFFu;
}

__host__ __device__ inline uint32_t lsb_to_half2(uint32_t w) {
    uint32_t even = squeeze_even_bits(w);       // elements 0,2,4,.. in bits 0..15
    uint32_t odd = squeeze_even_bits(w >> 1);   // elements 1,3,5,..
    return reverse16(even) | (reverse16(odd) << 16);
}

__host__ __device__ inline uint32_t half2_to_lsb(uint32_t h) {
    uint32_t even = reverse16(h & 0xFFFFu);
    uint32_t odd = reverse16(h >> 16);
    return spread_to_even_bits(even) | (spread_to_even_bits(odd) << 1);
}

__host__ __device__ inline uint32_t convert_order(uint32_t w, int from, int to) {
    if (from == to) return w;
    return from == NQ_LSB_FIRST ? lsb_to_half2(w) : half2_to_lsb(w);
}

}  // namespace nq
