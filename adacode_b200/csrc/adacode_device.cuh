// Device helpers shared by the float11 kernels (pack, unpack, fused decode attention): bit
// manipulation of bf16 words, zero-slot masks of packed code words, serialisation of a chunk's
// codes, block copies and the warp scan of escape counts.  Included inside an anonymous
// namespace by each .cu file.
#pragma once

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kCPT = 4;                          // chunks per thread per slab
constexpr int kSlabChunks = kThreads * kCPT;     // 1024
constexpr unsigned kFull = 0xFFFFFFFFu;

// ---------------------------------------------------------------------------------------
// bit helpers
// ---------------------------------------------------------------------------------------

// sign/mantissa bytes of two bf16 held in one 32-bit word, one byte per 16-bit lane
__device__ __forceinline__ uint32_t signmant_lanes(uint32_t w) {
    return ((w >> 8) & 0x00800080u) | (w & 0x007F007Fu);
}
// four sign/mantissa bytes from four consecutive bf16 (two words)
__device__ __forceinline__ uint32_t signmant4(uint32_t w0, uint32_t w1) {
    return __byte_perm(signmant_lanes(w0), signmant_lanes(w1), 0x6420);
}

// Mask with one bit at the least significant bit of each of the eight N-bit code slots.
template <int N>
struct SlotLsb;
template <>
struct SlotLsb<1> { static constexpr uint32_t v = 0xFFu; };
template <>
struct SlotLsb<2> { static constexpr uint32_t v = 0x5555u; };
template <>
struct SlotLsb<3> { static constexpr uint32_t v = 0x249249u; };
template <>
struct SlotLsb<4> { static constexpr uint32_t v = 0x11111111u; };

// Bit (at the slot LSB) for every code slot of the group word that holds code 0.
template <int N>
__device__ __forceinline__ uint32_t zero_slots(uint32_t g) {
    uint32_t m = g;
#pragma unroll
    for (int i = 1; i < N; ++i) m |= g >> i;
    return ~m & SlotLsb<N>::v;
}

// The eight slot bits of zero_slots<N>() (one per N-bit slot, at the slot's least significant bit)
// moved next to each other: slot j -> bit j, so element k of the group sits at bit 7 - k.
template <int N>
__device__ __forceinline__ uint32_t compress_slots(uint32_t z) {
    if constexpr (N == 1) {
        return z;
    } else if constexpr (N == 2) {
        z = (z | (z >> 1)) & 0x3333u;
        z = (z | (z >> 2)) & 0x0F0Fu;
        return (z | (z >> 4)) & 0xFFu;
    } else if constexpr (N == 3) {
        z = (z | (z >> 2)) & 0x0C30C3u;
        z = (z | (z >> 4)) & 0x00F00Fu;
        return (z | (z >> 8)) & 0xFFu;
    } else {
        z = (z | (z >> 3)) & 0x03030303u;
        z = (z | (z >> 6)) & 0x000F000Fu;
        return (z | (z >> 12)) & 0xFFu;
    }
}

// Eight exponent codes of eight consecutive bf16 (four words) as one group word:
// element k sits at bits [(7-k)*N, (8-k)*N).  Out-of-window exponents code as 0.
template <int N>
__device__ __forceinline__ uint32_t encode_group(const uint32_t w[4], int left) {
    constexpr uint32_t kMax = (1u << N) - 1u;
    uint32_t g = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t c0 = ((w[i] >> 7) & 0xFFu) - (uint32_t)left;
        uint32_t c1 = ((w[i] >> 23) & 0xFFu) - (uint32_t)left;
        c0 = c0 > kMax ? 0u : c0;
        c1 = c1 > kMax ? 0u : c1;
        g |= c0 << ((7 - 2 * i) * N);
        g |= c1 << ((6 - 2 * i) * N);
    }
    return g;
}

// In-window histogram: cnt[v] += number of slots of g holding code v (v = 1 .. 2^N-1).
template <int N>
__device__ __forceinline__ void count_codes(uint32_t g, uint32_t (&cnt)[1 << N]) {
    constexpr uint32_t M = SlotLsb<N>::v;
    uint32_t plane[N];
#pragma unroll
    for (int i = 0; i < N; ++i) plane[i] = (g >> i) & M;
#pragma unroll
    for (int v = 1; v < (1 << N); ++v) {
        uint32_t m = M;
#pragma unroll
        for (int i = 0; i < N; ++i) m &= ((v >> i) & 1) ? plane[i] : ~plane[i];
        cnt[v] += __popc(m);
    }
}

// ---------------------------------------------------------------------------------------
// code-byte (de)serialisation: a chunk of CH elements owns CH*N/8 bytes, each group of 8
// codes stored as an N-byte big-endian word
// ---------------------------------------------------------------------------------------

template <int N, int CH>
__device__ __forceinline__ void store_chunk_codes(uint8_t *s, const uint32_t g[CH / 8]) {
    if constexpr (CH == 16) {
        if constexpr (N == 1) {
            *reinterpret_cast<uint16_t *>(s) = (uint16_t)(g[0] | (g[1] << 8));
        } else if constexpr (N == 2) {
            *reinterpret_cast<uint32_t *>(s) = __byte_perm(g[0], g[1], 0x4501);
        } else if constexpr (N == 3) {
            const uint32_t lo = __byte_perm(g[0], g[1], 0x6012);
            const uint32_t hi = __byte_perm(g[1], 0u, 0x4401);
            uint16_t *p = reinterpret_cast<uint16_t *>(s);
            p[0] = (uint16_t)lo;
            p[1] = (uint16_t)(lo >> 16);
            p[2] = (uint16_t)hi;
        } else {
            uint2 v;
            v.x = __byte_perm(g[0], 0u, 0x0123);
            v.y = __byte_perm(g[1], 0u, 0x0123);
            *reinterpret_cast<uint2 *>(s) = v;
        }
    } else {
        if constexpr (N == 1) {
            s[0] = (uint8_t)g[0];
        } else if constexpr (N == 2) {
            *reinterpret_cast<uint16_t *>(s) = (uint16_t)__byte_perm(g[0], 0u, 0x4401);
        } else if constexpr (N == 3) {
            s[0] = (uint8_t)(g[0] >> 16);
            s[1] = (uint8_t)(g[0] >> 8);
            s[2] = (uint8_t)g[0];
        } else {
            *reinterpret_cast<uint32_t *>(s) = __byte_perm(g[0], 0u, 0x0123);
        }
    }
}

template <int N, int CH>
__device__ __forceinline__ void load_chunk_codes(const uint8_t *s, uint32_t g[CH / 8]) {
    if constexpr (CH == 16) {
        if constexpr (N == 1) {
            const uint32_t v = *reinterpret_cast<const uint16_t *>(s);
            g[0] = v & 0xFFu;
            g[1] = v >> 8;
        } else if constexpr (N == 2) {
            const uint32_t v = *reinterpret_cast<const uint32_t *>(s);
            g[0] = __byte_perm(v, 0u, 0x4401);
            g[1] = __byte_perm(v, 0u, 0x4423);
        } else if constexpr (N == 3) {
            const uint16_t *p = reinterpret_cast<const uint16_t *>(s);
            const uint32_t lo = (uint32_t)p[0] | ((uint32_t)p[1] << 16);
            const uint32_t hi = p[2];
            g[0] = __byte_perm(lo, 0u, 0x4012);
            g[1] = __byte_perm(lo, hi, 0x6345);
        } else {
            const uint2 v = *reinterpret_cast<const uint2 *>(s);
            g[0] = __byte_perm(v.x, 0u, 0x0123);
            g[1] = __byte_perm(v.y, 0u, 0x0123);
        }
    } else {
        if constexpr (N == 1) {
            g[0] = s[0];
        } else if constexpr (N == 2) {
            g[0] = __byte_perm((uint32_t) * reinterpret_cast<const uint16_t *>(s), 0u, 0x4401);
        } else if constexpr (N == 3) {
            g[0] = ((uint32_t)s[0] << 16) | ((uint32_t)s[1] << 8) | s[2];
        } else {
            g[0] = __byte_perm(*reinterpret_cast<const uint32_t *>(s), 0u, 0x0123);
        }
    }
}

// Copy `bytes` bytes between shared and global memory with the whole block, 16 bytes at a
// time when both ends allow it.
__device__ __forceinline__ void block_copy_out(uint8_t *dst, const uint8_t *s_src, int bytes) {
    if ((((uintptr_t)dst | (uintptr_t)bytes) & 15) == 0) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(s_src);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
        for (int i = threadIdx.x; i < bytes / 16; i += kThreads) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < bytes; i += kThreads) dst[i] = s_src[i];
    }
}
__device__ __forceinline__ void block_copy_in(uint8_t *s_dst, const uint8_t *src, int bytes) {
    if ((((uintptr_t)src | (uintptr_t)bytes) & 15) == 0) {
        const uint4 *g4 = reinterpret_cast<const uint4 *>(src);
        uint4 *s4 = reinterpret_cast<uint4 *>(s_dst);
        for (int i = threadIdx.x; i < bytes / 16; i += kThreads) s4[i] = __ldg(g4 + i);
    } else {
        for (int i = threadIdx.x; i < bytes; i += kThreads) s_dst[i] = src[i];
    }
}

// Inclusive warp scans of four counters per lane, walked in (k, lane) order.  Counters are
// at most 16, so two share one register as 16-bit fields.  On return incl[k] is the
// inclusive rank of (k, lane) within the warp's 4x32 chunks; the return value is the total.
__device__ __forceinline__ int warp_scan4(const int cnt[kCPT], int incl[kCPT]) {
    uint32_t a = (uint32_t)cnt[0] | ((uint32_t)cnt[1] << 16);
    uint32_t b = (uint32_t)cnt[2] | ((uint32_t)cnt[3] << 16);
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t ua = __shfl_up_sync(kFull, a, d);
        const uint32_t ub = __shfl_up_sync(kFull, b, d);
        if (lane >= d) {
            a += ua;
            b += ub;
        }
    }
    const uint32_t ta = __shfl_sync(kFull, a, 31);
    const uint32_t tb = __shfl_sync(kFull, b, 31);
    const int t0 = ta & 0xFFFF, t1 = ta >> 16, t2 = tb & 0xFFFF, t3 = tb >> 16;
    incl[0] = (int)(a & 0xFFFF);
    incl[1] = (int)(a >> 16) + t0;
    incl[2] = (int)(b & 0xFFFF) + t0 + t1;
    incl[3] = (int)(b >> 16) + t0 + t1 + t2;
    return t0 + t1 + t2 + t3;
}

// ---- table-driven decode -------------------------------------------------------------------
// The integer pipe (half the rate of the issue slots) is what limits these kernels, so the
// per-element shifts, masks and adds of the decode are replaced by one shared-memory lookup per
// pair (or quadruple, or octet) of codes: the table maps a run of packed code bits to the
// finished exponent fields of the corresponding bf16 pairs, `(e0 << 7) | (e1 << 23)`, with the
// window's left edge already added (and 0 for code 0).  Index width: 8 bits for N = 1, 2, 4; 6 bits for N = 3.
template <int N>
struct DecodeLut {
    static constexpr int index_bits = (N == 3) ? 6 : 8;
    static constexpr int elems = index_bits / N;          // elements covered by one lookup
    static constexpr int words = elems / 2;               // 32-bit pair words per entry
    static constexpr int entries = 1 << index_bits;
};

__device__ __forceinline__ void build_decode_lut(uint32_t *lut, int N, int left, int n_threads) {
    const int index_bits = (N == 3) ? 6 : 8;
    const int words = (index_bits / N) / 2;
    const int total = (1 << index_bits) * words;
    const uint32_t mask = (1u << N) - 1u;
    for (int w = threadIdx.x; w < total; w += n_threads) {
        const uint32_t e = (uint32_t)(w / words), p = (uint32_t)(w % words);
        const uint32_t c_even = (e >> (index_bits - (2 * p + 1) * N)) & mask;
        const uint32_t c_odd = (e >> (index_bits - (2 * p + 2) * N)) & mask;
        // code 0 (an escape) decodes to exponent field 0, so that the escaped exponent can be OR-ed in
        const uint32_t e_even = c_even ? ((c_even + (uint32_t)left) & 0xFFu) : 0u;
        const uint32_t e_odd = c_odd ? ((c_odd + (uint32_t)left) & 0xFFu) : 0u;
        lut[w] = (e_even << 7) | (e_odd << 23);
    }
}

// Exponent fields of the four bf16 pairs of group word g (element 0 in the most significant bits).
template <int N>
__device__ __forceinline__ void decode_group(const uint32_t *lut, uint32_t g, uint32_t (&ew)[4]) {
    if constexpr (N == 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) ew[i] = lut[(g >> (24 - 8 * i)) & 0xFFu];
    } else if constexpr (N == 3) {
#pragma unroll
        for (int i = 0; i < 4; ++i) ew[i] = lut[(g >> (18 - 6 * i)) & 0x3Fu];
    } else if constexpr (N == 2) {
        const uint2 hi = reinterpret_cast<const uint2 *>(lut)[(g >> 8) & 0xFFu];
        const uint2 lo = reinterpret_cast<const uint2 *>(lut)[g & 0xFFu];
        ew[0] = hi.x, ew[1] = hi.y, ew[2] = lo.x, ew[3] = lo.y;
    } else {
        const uint4 v = reinterpret_cast<const uint4 *>(lut)[g & 0xFFu];
        ew[0] = v.x, ew[1] = v.y, ew[2] = v.z, ew[3] = v.w;
    }
}

