// Pack / layout kernels.  All integer work, bit-exact with the reference's
// PyTorch packers (src/nanoquant/kernel/utils.py in the reference project):
//
//   rows layout    int32 [rows, ceil(cols/32)], bit order lsb_first or half2
//   marlin layout  int32 [in/16, out/2], one word = the B fragments of one lane
//   tile layout    the runtime layout of the GEMV kernel here, see nq_rows_to_tiles
//
// Each thread produces whole output words so that stores are coalesced; the
// kernels are bound by the bytes they read and write.
#include "nq_common.cuh"

namespace nq {

constexpr int kPackThreads = 256;

static inline unsigned grid_for(int64_t n, int threads) {
    int64_t g = (n + threads - 1) / threads;
    const int64_t cap = 148LL * 64;  // grid-stride beyond this
    return static_cast<unsigned>(g < 1 ? 1 : (g > cap ? cap : g));
}

// sign bits of four int8 values held in one register -> 4-bit field (byte b -> bit b)
__device__ __forceinline__ uint32_t sign_nibble(uint32_t v) {
    uint32_t x = (v >> 7) & 0x01010101u;
    return (x * 0x01020408u) >> 24;  // gathers bits 0,8,16,24 into bits 0..3
}

// 4-bit field -> bit b placed at position 8*b
__device__ __forceinline__ uint32_t spread_nibble(uint32_t n) {
    return ((n & 0xFu) * 0x00204081u) & 0x01010101u;
}

// ---------------------------------------------------------------------------
// rows layout
// ---------------------------------------------------------------------------
__global__ void pack_rows_kernel(const int8_t* __restrict__ w, uint32_t* __restrict__ out,
                                 int64_t rows, int64_t cols, int64_t words, int order, bool vec) {
    const int64_t total = rows * words;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / words, wi = i - r * words;
        const int64_t c0 = wi * 32;
        const int8_t* src = w + r * cols + c0;
        uint32_t bits = 0;
        if (vec && c0 + 32 <= cols) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(src));
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(src) + 1);
            bits = sign_nibble(a.x) | (sign_nibble(a.y) << 4) | (sign_nibble(a.z) << 8) |
                   (sign_nibble(a.w) << 12) | (sign_nibble(b.x) << 16) | (sign_nibble(b.y) << 20) |
                   (sign_nibble(b.z) << 24) | (sign_nibble(b.w) << 28);
        } else {
            const int n = (int)((cols - c0) < 32 ? (cols - c0) : 32);
            for (int k = 0; k < n; ++k) bits |= (uint32_t)(src[k] < 0) << k;  // padding stays +1 (bit 0)
        }
        out[i] = convert_order(bits, NQ_LSB_FIRST, order);
    }
}

__global__ void unpack_rows_kernel(const uint32_t* __restrict__ packed, int8_t* __restrict__ w,
                                   int64_t rows, int64_t cols, int64_t words, int order, bool vec) {
    const int64_t total = rows * words;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / words, wi = i - r * words;
        const int64_t c0 = wi * 32;
        const uint32_t bits = convert_order(packed[i], order, NQ_LSB_FIRST);
        int8_t* dst = w + r * cols + c0;
        if (vec && c0 + 32 <= cols) {
            uint32_t v[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                // bit b of the nibble -> byte b; +1 = 0x01, -1 = 0xFF  (1 - 2*bit)
                const uint32_t s = spread_nibble(bits >> (4 * k));
                v[k] = 0x01010101u + s * 0xFEu;
            }
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(v[4], v[5], v[6], v[7]);
        } else {
            const int n = (int)((cols - c0) < 32 ? (cols - c0) : 32);
            for (int k = 0; k < n; ++k) dst[k] = ((bits >> k) & 1u) ? (int8_t)-1 : (int8_t)1;
        }
    }
}

// The same two conversions for matrices of whole 32-column words at a 16-byte aligned address, with every global
// access of a warp contiguous: the dense side moves in 512-byte pieces (one 16-byte piece per lane), the packed
// side in 128-byte pieces (one word per lane), and the lanes trade their halves with shuffles.  A warp handles
// 32 consecutive words (1 KB of weights) per step; `n_words` is a multiple of 32 here, the tail goes to the
// word-per-thread kernels above.
__global__ void __launch_bounds__(256) pack_rows_warp_kernel(const uint4* __restrict__ w, uint32_t* __restrict__ out,
                                                             int64_t n_words, int order) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = ((blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5) * 32; base < n_words; base += warps * 32) {
        // piece p (16 weights) of this step belongs to word base + p/2, half p & 1
        const uint4 a = __ldcs(w + base * 2 + lane), b = __ldcs(w + base * 2 + 32 + lane);
        const uint32_t ha = sign_nibble(a.x) | (sign_nibble(a.y) << 4) | (sign_nibble(a.z) << 8) | (sign_nibble(a.w) << 12);
        const uint32_t hb = sign_nibble(b.x) | (sign_nibble(b.y) << 4) | (sign_nibble(b.z) << 8) | (sign_nibble(b.w) << 12);
        // lane L wants word base + L: its halves are pieces 2L and 2L + 1, i.e. lanes 2(L & 15) and +1 of load a (L < 16) or b
        const int src = 2 * (lane & 15);
        const uint32_t a_lo = __shfl_sync(0xffffffffu, ha, src), a_hi = __shfl_sync(0xffffffffu, ha, src + 1);
        const uint32_t b_lo = __shfl_sync(0xffffffffu, hb, src), b_hi = __shfl_sync(0xffffffffu, hb, src + 1);
        const uint32_t bits = lane < 16 ? (a_lo | (a_hi << 16)) : (b_lo | (b_hi << 16));
        out[base + lane] = convert_order(bits, NQ_LSB_FIRST, order);
    }
}

__global__ void __launch_bounds__(256) unpack_rows_warp_kernel(const uint32_t* __restrict__ packed, uint4* __restrict__ w,
                                                               int64_t n_words, int order) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = ((blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5) * 32; base < n_words; base += warps * 32) {
        const uint32_t mine = convert_order(__ldcs(packed + base + lane), order, NQ_LSB_FIRST);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            // piece 32k + lane: word base + 16k + lane/2, half lane & 1
            const uint32_t word = __shfl_sync(0xffffffffu, mine, 16 * k + (lane >> 1));
            const uint32_t h = (word >> (16 * (lane & 1))) & 0xFFFFu;
            uint32_t v[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) v[q] = 0x01010101u + spread_nibble(h >> (4 * q)) * 0xFEu;   // +1 = 0x01, -1 = 0xFF
            __stcs(w + base * 2 + 32 * k + lane, make_uint4(v[0], v[1], v[2], v[3]));
        }
    }
}

__global__ void reorder_words_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                     int64_t n, int from, int to) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = convert_order(in[i], from, to);
}
// the same with 16-byte accesses (n4 groups of four words, both pointers 16-byte aligned)
__global__ void reorder_words4_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int64_t n4, int from, int to) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 v = __ldg(in + i);
        out[i] = make_uint4(convert_order(v.x, from, to), convert_order(v.y, from, to), convert_order(v.z, from, to),
                            convert_order(v.w, from, to));
    }
}

// ---------------------------------------------------------------------------
// marlin layout.  out = 64*to + 16*o16 + 8*o8 + o1, in = 16*tr + 8*r8 + 2*r2 + r1
//   word (tr, 32*to + 4*o1 + r2), bit 15 - 4*o16 - 2*o8 - r8 + 16*r1
// ---------------------------------------------------------------------------
__global__ void pack_marlin_kernel(const int8_t* __restrict__ w, uint32_t* __restrict__ B,
                                   int64_t out_f, int64_t in_f) {
    const int64_t ncol = out_f / 2, total = (in_f / 16) * ncol;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tr = i / ncol, col = i - tr * ncol;
        const int64_t to = col >> 5;
        const int o1 = (int)(col & 31) >> 2, r2 = (int)(col & 3);
        uint32_t bits = 0;
#pragma unroll
        for (int o16 = 0; o16 < 4; ++o16)
#pragma unroll
            for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
                for (int r8 = 0; r8 < 2; ++r8) {
                    const int64_t o = 64 * to + 16 * o16 + 8 * o8 + o1;
                    const int64_t k = 16 * tr + 8 * r8 + 2 * r2;
                    const int8_t* p = w + o * in_f + k;
                    const int pos = 15 - 4 * o16 - 2 * o8 - r8;
                    bits |= (uint32_t)(p[0] < 0) << pos;
                    bits |= (uint32_t)(p[1] < 0) << (pos + 16);
                }
        B[i] = bits;
    }
}

// The same through shared memory: a CTA stages 64 output rows x 128 input columns with 16-byte row loads (a row
// segment of 128 bytes is one coalesced request) and every thread assembles one word of the 8 x 32 words of the
// tile from it.  The direct kernel above reads two single bytes per bit pair at a stride of in_f bytes.
constexpr int kMarlinKT = 128;              // input columns per CTA
constexpr int kMarlinPitch = kMarlinKT + 16;
__global__ void __launch_bounds__(256) pack_marlin_staged_kernel(const int8_t* __restrict__ w, uint32_t* __restrict__ B,
                                                                 int64_t out_f, int64_t in_f) {
    __shared__ __align__(16) int8_t tile[64 * kMarlinPitch];
    const int64_t to = blockIdx.x, k0 = (int64_t)blockIdx.y * kMarlinKT;
    const int t = threadIdx.x;
    for (int idx = t; idx < 64 * (kMarlinKT / 16); idx += 256) {
        const int row = idx / (kMarlinKT / 16), seg = idx % (kMarlinKT / 16);
        if (k0 + 16 * seg < in_f)      // in_f is a multiple of 16: a segment is inside the row or beyond it as a whole
            *reinterpret_cast<uint4*>(tile + row * kMarlinPitch + 16 * seg) =
                __ldg(reinterpret_cast<const uint4*>(w + (64 * to + row) * in_f + k0 + 16 * seg));
    }
    __syncthreads();
    const int trl = t >> 5, colw = t & 31;
    if (k0 + 16 * trl >= in_f) return;
    const int o1 = colw >> 2, r2 = colw & 3;
    uint32_t bits = 0;
#pragma unroll
    for (int o16 = 0; o16 < 4; ++o16)
#pragma unroll
        for (int o8 = 0; o8 < 2; ++o8)
#pragma unroll
            for (int r8 = 0; r8 < 2; ++r8) {
                // the two weights of a bit pair are neighbours: one 16-bit load, sign bits 7 and 15 -> pos and pos + 16
                const uint32_t h = *reinterpret_cast<const uint16_t*>(tile + (16 * o16 + 8 * o8 + o1) * kMarlinPitch +
                                                                      16 * trl + 8 * r8 + 2 * r2);
                const int pos = 15 - 4 * o16 - 2 * o8 - r8;
                bits |= (((h >> 7) & 1u) | ((h << 1) & 0x10000u)) << pos;
            }
    B[(k0 / 16 + trl) * (out_f / 2) + 32 * to + colw] = bits;
}

__global__ void marlin_to_rows_kernel(const uint32_t* __restrict__ B, uint32_t* __restrict__ packed,
                                      int64_t out_f, int64_t in_f, int order) {
    const int64_t words = in_f / 32, total = out_f * words, ncol = out_f / 2;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / words, wi = i - o * words;
        const int64_t to = o >> 6;
        const int o16 = (int)(o >> 4) & 3, o8 = (int)(o >> 3) & 1, o1 = (int)o & 7;
        uint32_t bits = 0;
#pragma unroll
        for (int t = 0; t < 2; ++t) {  // two k-tiles of 16 per 32-column word
            const int64_t tr = wi * 2 + t;
#pragma unroll
            for (int r2 = 0; r2 < 4; ++r2) {
                const uint32_t src = B[tr * ncol + 32 * to + 4 * o1 + r2];
#pragma unroll
                for (int r8 = 0; r8 < 2; ++r8)
#pragma unroll
                    for (int r1 = 0; r1 < 2; ++r1) {
                        const int pos = 15 - 4 * o16 - 2 * o8 - r8 + 16 * r1;
                        const int k = 16 * t + 8 * r8 + 2 * r2 + r1;
                        bits |= ((src >> pos) & 1u) << k;
                    }
            }
        }
        packed[i] = convert_order(bits, NQ_LSB_FIRST, order);
    }
}

// kind 0: groups of 16, new[4b+2a+c] = old[8a+2b+c]; kind 1: groups of 32, new[8b+2a+c] = old[8a+2b+c]
__global__ void permute_scale16_kernel(const uint16_t* __restrict__ s, uint16_t* __restrict__ out,
                                       int64_t n, int kind, int inverse) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t base;
        int p, a, b, c, src;
        if (kind == 0) {
            base = i & ~15LL; p = (int)(i & 15);
            b = p >> 2; a = (p >> 1) & 1; c = p & 1;   // p = 4b + 2a + c
            src = 8 * a + 2 * b + c;
        } else {
            base = i & ~31LL; p = (int)(i & 31);
            b = p >> 3; a = (p >> 1) & 3; c = p & 1;   // p = 8b + 2a + c
            src = 8 * a + 2 * b + c;
        }
        if (!inverse) out[i] = s[base + src];
        else out[base + src] = s[i];
    }
}

// ---------------------------------------------------------------------------
// tile layout of the GEMV kernel
//
// A tile covers 16 rows x 256 columns and is stored as 32 lanes x uint4 (512 B),
// tiles ordered [row_group][chunk].  Lane l = 4*g + q holds
//   .x: row g,   columns half h=0      .y: row g+8, h=0
//   .z: row g,   h=1                   .w: row g+8, h=1
// and inside a word the weight of column 32*j + 16*h + 4*q + b (of the chunk)
// sits at bit 8*b + j.  `word & (0x01010101 << j)` is then directly the int8
// A-fragment register of an m16n8k32 MMA over columns [32j, 32j+32) with values
// {0, 2^j} (j = 7: {0, -128}).  Rows and columns beyond the matrix are +1 (bit 0).
// ---------------------------------------------------------------------------
// Through shared memory: a work item is one row group (16 rows) by eight chunks (64 words per row); a block
// reads the 16 row pieces of 256 bytes with contiguous loads and writes eight whole tiles (one uint4 per thread).
// (One thread per output lane reading its 16 words straight from global memory touches a 32-byte sector per word.)
// Blocks stride over the items and load the next item's words into registers before they convert the current one.
__global__ void __launch_bounds__(256) rows_to_tiles_staged_kernel(const uint32_t* __restrict__ packed, uint4* __restrict__ tiles,
                                                                   int64_t rows, int64_t words, int64_t chunks, int64_t cblocks,
                                                                   int64_t items, int order) {
    __shared__ uint32_t s[16][65];
    const int cl = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    uint32_t nxt[4];
    auto fetch = [&](int64_t item) {
        const int64_t rg = item / cblocks, c0 = (item - rg * cblocks) * 8;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x + 256 * k, r = i >> 6, wl = i & 63;
            const int64_t gr = rg * 16 + r, gw = c0 * 8 + wl;
            nxt[k] = (gr < rows && gw < words) ? __ldcs(packed + gr * words + gw) : 0u;
        }
    };
    int64_t item = blockIdx.x;
    if (item < items) fetch(item);
    for (; item < items; item += gridDim.x) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = threadIdx.x + 256 * k;
            s[i >> 6][i & 63] = convert_order(nxt[k], order, NQ_LSB_FIRST);   // padding words are 0 in either order
        }
        __syncthreads();
        if (item + gridDim.x < items) fetch(item + gridDim.x);
        const int64_t rg = item / cblocks, c0 = (item - rg * cblocks) * 8;
        if (c0 + cl < chunks) {
            uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
            for (int half_row = 0; half_row < 2; ++half_row)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t src = s[g + 8 * half_row][cl * 8 + j];
                    o[half_row] |= spread_nibble(src >> (4 * q)) << j;           // h = 0
                    o[2 + half_row] |= spread_nibble(src >> (16 + 4 * q)) << j;  // h = 1
                }
            __stcs(tiles + ((rg * chunks + c0 + cl) << 5) + lane, make_uint4(o[0], o[1], o[2], o[3]));
        }
        __syncthreads();
    }
}

__global__ void tiles_to_rows_kernel(const uint4* __restrict__ tiles, uint32_t* __restrict__ packed,
                                     int64_t rows, int64_t words, int64_t chunks, int order) {
    const int64_t total = rows * words;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / words, wi = i - r * words;
        const int64_t rg = r >> 4, c = wi >> 3;
        const int g = (int)(r & 7), half_row = (int)(r >> 3) & 1, j = (int)(wi & 7);
        uint32_t bits = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 t = tiles[(rg * chunks + c) * 32 + 4 * g + q];
            const uint32_t lo = half_row ? t.y : t.x, hi = half_row ? t.w : t.z;
            const uint32_t nlo = (((lo >> j) & 0x01010101u) * 0x01020408u) >> 24;
            const uint32_t nhi = (((hi >> j) & 0x01010101u) * 0x01020408u) >> 24;
            bits |= (nlo & 0xFu) << (4 * q);
            bits |= (nhi & 0xFu) << (16 + 4 * q);
        }
        packed[i] = convert_order(bits, NQ_LSB_FIRST, order);
    }
}

// gcd(n, 32) for n > 0: the largest power of two up to 32 that divides n
static int64_t gcd32(int64_t n) {
    int64_t g = 1;
    while (g < 32 && n % (2 * g) == 0) g *= 2;
    return g;
}

static int check_order(int o) { return (o == NQ_LSB_FIRST || o == NQ_HALF2) ? NQ_OK : NQ_ERR_DTYPE; }

}  // namespace nq

using namespace nq;

extern "C" {

int nq_pack_rows(const int8_t* w, int32_t* packed, int64_t rows, int64_t cols, int bit_order,
                 nq_stream_t stream) {
    if (rows < 0 || cols < 0) return NQ_ERR_SHAPE;
    if (check_order(bit_order) != NQ_OK) return NQ_ERR_DTYPE;
    if (rows == 0 || cols == 0) return NQ_OK;
    if (!w || !packed) return NQ_ERR_NULL;
    const int64_t words = (cols + 31) / 32;
    const bool vec = (cols % 16 == 0) && aligned16(w);
    // whole words at an aligned address: the rows form one run of words; the leading rows whose words are a multiple
    // of 32 go to the warp-contiguous kernel, the remaining rows to the word-per-thread kernel
    int64_t done_rows = 0;
    if (cols % 32 == 0 && aligned16(w)) {
        const int64_t step = 32 / gcd32(words), head_rows = rows / step * step, head = head_rows * words;
        if (head > 0) {
            pack_rows_warp_kernel<<<grid_for(head, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
                reinterpret_cast<const uint4*>(w), reinterpret_cast<uint32_t*>(packed), head, bit_order);
            NQ_LAUNCH_CHECK();
            done_rows = head_rows;
        }
    }
    if (done_rows < rows) {
        pack_rows_kernel<<<grid_for((rows - done_rows) * words, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
            w + done_rows * cols, reinterpret_cast<uint32_t*>(packed) + done_rows * words, rows - done_rows, cols, words,
            bit_order, vec);
        NQ_LAUNCH_CHECK();
    }
    return NQ_OK;
}

int nq_unpack_rows(const int32_t* packed, int8_t* w, int64_t rows, int64_t cols, int bit_order,
                   nq_stream_t stream) {
    if (rows < 0 || cols < 0) return NQ_ERR_SHAPE;
    if (check_order(bit_order) != NQ_OK) return NQ_ERR_DTYPE;
    if (rows == 0 || cols == 0) return NQ_OK;
    if (!w || !packed) return NQ_ERR_NULL;
    const int64_t words = (cols + 31) / 32;
    const bool vec = (cols % 16 == 0) && aligned16(w);
    int64_t done_rows = 0;
    if (cols % 32 == 0 && aligned16(w)) {   // see nq_pack_rows
        const int64_t step = 32 / gcd32(words), head_rows = rows / step * step, head = head_rows * words;
        if (head > 0) {
            unpack_rows_warp_kernel<<<grid_for(head, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
                reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<uint4*>(w), head, bit_order);
            NQ_LAUNCH_CHECK();
            done_rows = head_rows;
        }
    }
    if (done_rows < rows) {
        unpack_rows_kernel<<<grid_for((rows - done_rows) * words, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
            reinterpret_cast<const uint32_t*>(packed) + done_rows * words, w + done_rows * cols, rows - done_rows, cols, words,
            bit_order, vec);
        NQ_LAUNCH_CHECK();
    }
    return NQ_OK;
}

int nq_reorder_words(const int32_t* in, int32_t* out, int64_t n_words, int order_in, int order_out,
                     nq_stream_t stream) {
    if (n_words < 0) return NQ_ERR_SHAPE;
    if (check_order(order_in) != NQ_OK || check_order(order_out) != NQ_OK) return NQ_ERR_DTYPE;
    if (n_words == 0) return NQ_OK;
    if (!in || !out) return NQ_ERR_NULL;
    if (n_words % 4 == 0 && aligned16(in) && aligned16(out))
        reorder_words4_kernel<<<grid_for(n_words / 4, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
            reinterpret_cast<const uint4*>(in), reinterpret_cast<uint4*>(out), n_words / 4, order_in, order_out);
    else
        reorder_words_kernel<<<grid_for(n_words, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
            reinterpret_cast<const uint32_t*>(in), reinterpret_cast<uint32_t*>(out), n_words, order_in, order_out);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

int nq_pack_marlin(const int8_t* w, int32_t* B, int64_t out_f, int64_t in_f, nq_stream_t stream) {
    if (out_f < 0 || in_f < 0 || out_f % 64 || in_f % 16) return NQ_ERR_SHAPE;
    if (out_f == 0 || in_f == 0) return NQ_OK;
    if (!w || !B) return NQ_ERR_NULL;
    const int64_t kblocks = (in_f + kMarlinKT - 1) / kMarlinKT;
    if (aligned16(w) && out_f / 64 <= 0x7FFFFFFF && kblocks <= 65535)
        pack_marlin_staged_kernel<<<dim3((unsigned)(out_f / 64), (unsigned)kblocks), 256, 0, as_stream(stream)>>>(
            w, reinterpret_cast<uint32_t*>(B), out_f, in_f);
    else
        pack_marlin_kernel<<<grid_for((in_f / 16) * (out_f / 2), kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
            w, reinterpret_cast<uint32_t*>(B), out_f, in_f);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

int nq_marlin_to_rows(const int32_t* B, int32_t* packed, int64_t out_f, int64_t in_f, int bit_order,
                      nq_stream_t stream) {
    if (out_f < 0 || in_f < 0 || out_f % 64 || in_f % 32) return NQ_ERR_SHAPE;
    if (check_order(bit_order) != NQ_OK) return NQ_ERR_DTYPE;
    if (out_f == 0 || in_f == 0) return NQ_OK;
    if (!B || !packed) return NQ_ERR_NULL;
    marlin_to_rows_kernel<<<grid_for(out_f * (in_f / 32), kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint32_t*>(B), reinterpret_cast<uint32_t*>(packed), out_f, in_f, bit_order);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

int nq_permute_scale16(const void* s, void* out, int64_t n, int kind, int inverse, nq_stream_t stream) {
    if (kind != 0 && kind != 1) return NQ_ERR_DTYPE;
    if (n < 0 || n % (kind == 0 ? 16 : 32)) return NQ_ERR_SHAPE;
    if (n == 0) return NQ_OK;
    if (!s || !out) return NQ_ERR_NULL;
    if (s == out) return NQ_ERR_UNSUPPORTED;  // not an in-place permutation
    permute_scale16_kernel<<<grid_for(n, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
        static_cast<const uint16_t*>(s), static_cast<uint16_t*>(out), n, kind, inverse);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

size_t nq_tiles_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return (size_t)((rows + 15) / 16) * (size_t)((cols + 255) / 256) * 512;
}

int nq_rows_to_tiles(const int32_t* packed, void* tiles, int64_t rows, int64_t cols, int bit_order,
                     nq_stream_t stream) {
    if (rows <= 0 || cols <= 0) return NQ_ERR_SHAPE;
    if (check_order(bit_order) != NQ_OK) return NQ_ERR_DTYPE;
    if (!packed || !tiles) return NQ_ERR_NULL;
    if (!aligned16(tiles)) return NQ_ERR_ALIGN;
    const int64_t words = (cols + 31) / 32, rgs = (rows + 15) / 16, chunks = (cols + 255) / 256;
    const int64_t cblocks = (chunks + 7) / 8, items = rgs * cblocks;
    const int64_t resident = (int64_t)sm_count() * 8;   // 256-thread blocks that are resident at once
    rows_to_tiles_staged_kernel<<<(unsigned)(items < resident ? items : resident), 256, 0, as_stream(stream)>>>(
        reinterpret_cast<const uint32_t*>(packed), static_cast<uint4*>(tiles), rows, words, chunks, cblocks, items, bit_order);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

int nq_tiles_to_rows(const void* tiles, int32_t* packed, int64_t rows, int64_t cols, int bit_order,
                     nq_stream_t stream) {
    if (rows <= 0 || cols <= 0) return NQ_ERR_SHAPE;
    if (check_order(bit_order) != NQ_OK) return NQ_ERR_DTYPE;
    if (!packed || !tiles) return NQ_ERR_NULL;
    if (!aligned16(tiles)) return NQ_ERR_ALIGN;
    const int64_t words = (cols + 31) / 32, chunks = (cols + 255) / 256;
    tiles_to_rows_kernel<<<grid_for(rows * words, kPackThreads), kPackThreads, 0, as_stream(stream)>>>(
        static_cast<const uint4*>(tiles), reinterpret_cast<uint32_t*>(packed), rows, words, chunks, bit_order);
    NQ_LAUNCH_CHECK();
    return NQ_OK;
}

}  // extern "C"
