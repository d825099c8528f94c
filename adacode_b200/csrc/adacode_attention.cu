// Fused unpack + single-query ("decode") attention over a float11-packed KV cache.
//
// The packed planes are read straight from HBM (1 + n/8 + p bytes per cached element instead of
// 2 for dense bf16), decoded tile by tile into shared memory, and consumed there: scores against
// the G query heads that share a KV head, online softmax in fp32, weighted sum of the decoded V
// tile.  The cache is split along the sequence (flash-decoding): grid = (splits, B * Hkv), each
// CTA owns a run of 128-token tiles of one (batch, kv head) and leaves (max, sum, numerator)
// partials that a second kernel combines.
//
// The reference has no such kernel (its attention path materialises dense K/V first; the module
// its validation script imports, ops/kv_attention.py, is absent from its tree), so numerics are
// checked against an fp32 PyTorch attention over the dense cache.
#include <cuda_runtime.h>
#include <stdint.h>

#include "adacode.h"

#include <stdlib.h>

namespace {

#include "adacode_device.cuh"
#define ADACODE_PIPELINE_UNPACK_ONLY
#include "adacode_pipeline.cuh"

constexpr int kAttnThreads = 128;
constexpr int kTileTokens = 128;
constexpr int kMaxGroup = 8;      // query heads per KV head
constexpr int kMaxD = 128;

struct AttnArgs {
    const uint16_t *q;            // [B][Hq][D]
    long long q_sb, q_sh;
    const adacode_segment *kseg, *vseg;
    int n_seg;
    const uint16_t *k_tail, *v_tail;   // dense residual [B][Hkv][tail_len][D]
    int tail_len;
    long long t_sb, t_sh, t_ss;
    int B, Hq, Hkv, G, D;
    float scale;
    int n_splits;
    float *part_o;                // [B*Hkv][splits][G][D]
    float *part_ml;               // [B*Hkv][splits][G][2]
    int32_t *status;
};

struct AttnSmem {
    alignas(16) uint8_t sm[kTileTokens * kMaxD];          // staged sign/mantissa plane of one tile
    alignas(16) uint8_t codes[kTileTokens * kMaxD / 2];   // staged code plane
    alignas(16) uint16_t tile[kTileTokens * (kMaxD + 2)]; // decoded (or dense) tile, rows padded by 2
    alignas(16) float q[kMaxGroup][kMaxD];
    alignas(16) float p[kTileTokens][kMaxGroup];       // softmax numerators, [token][query head]
    alignas(16) uint32_t lut[2][1024];                    // decode tables: [0] keys, [1] values
    int lut_left[2], lut_nbits[2];
    float red[kMaxGroup][4];
    int scan[4];
};

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Decode tile `bh` of one packed segment into s.tile (row stride D + 2 elements).
template <int N>
__device__ __forceinline__ void decode_tile(AttnSmem &s, const adacode_segment &sg, int bh, int D, const uint32_t *lut,
                                            int32_t *status) {
    constexpr int CB = 2 * N;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile_elems = kTileTokens * D;
    const int chunks = tile_elems >> 4;
    const int per_thread = chunks / kAttnThreads;             // 8 at D = 128, 4 at D = 64
    const uint8_t *gsm = sg.sign_mant + (long long)bh * tile_elems;
    const uint8_t *gcd = sg.codes + (long long)bh * (tile_elems * N / 8);
    // stage both planes with coalesced 16-byte loads
    for (int i = tid; i < tile_elems / 16; i += kAttnThreads)
        reinterpret_cast<uint4 *>(s.sm)[i] = __ldg(reinterpret_cast<const uint4 *>(gsm) + i);
    for (int i = tid; i < tile_elems * N / 128; i += kAttnThreads)
        reinterpret_cast<uint4 *>(s.codes)[i] = __ldg(reinterpret_cast<const uint4 *>(gcd) + i);
    __syncthreads();

    // pass 1: escapes in this thread's run of chunks, then an exclusive scan over the block
    const int c0 = tid * per_thread;
    int cnt = 0;
    for (int k = 0; k < per_thread; ++k) {
        uint32_t g[2];
        load_chunk_codes<N, 16>(s.codes + (c0 + k) * CB, g);
        cnt += __popc(zero_slots<N>(g[0])) + __popc(zero_slots<N>(g[1]));
    }
    int x = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int u = __shfl_up_sync(kFull, x, d);
        if (lane >= d) x += u;
    }
    if (lane == 31) s.scan[warp] = x;
    __syncthreads();
    int rank = x - cnt;
    for (int i = 0; i < warp; ++i) rank += s.scan[i];
    const long long esc0 = bh > 0 ? sg.tile_base[bh - 1] : 0;

    // pass 2: decode, write the padded rows, patch escapes
    const int row_stride = D + 2;
    for (int k = 0; k < per_thread; ++k) {
        const int c = c0 + k;
        uint32_t g[2];
        load_chunk_codes<N, 16>(s.codes + c * CB, g);
        const uint4 sv = *reinterpret_cast<const uint4 *>(s.sm + c * 16);
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        const int e0 = c * 16;
        const int row = e0 / D, col = e0 - row * D;
        uint32_t *dst = reinterpret_cast<uint32_t *>(s.tile + row * row_stride + col);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t ew[4];
            decode_group<N>(lut, g[q], ew);
            const uint32_t s0 = sw[2 * q], s1 = sw[2 * q + 1];
            dst[4 * q + 0] = ew[0] | (__byte_perm(s0, 0u, 0x1100) & 0x807F807Fu);
            dst[4 * q + 1] = ew[1] | (__byte_perm(s0, 0u, 0x3322) & 0x807F807Fu);
            dst[4 * q + 2] = ew[2] | (__byte_perm(s1, 0u, 0x1100) & 0x807F807Fu);
            dst[4 * q + 3] = ew[3] | (__byte_perm(s1, 0u, 0x3322) & 0x807F807Fu);
        }
        uint16_t *row16 = reinterpret_cast<uint16_t *>(dst);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t z = zero_slots<N>(g[q]);
            while (z) {
                const int pos = 31 - __clz(z);
                z ^= 1u << pos;
                const int el = q * 8 + 7 - pos / N;
                uint32_t e = 0;
                const long long idx = esc0 + rank;
                if (idx < sg.escapes_len) e = sg.escapes[idx];
                else atomicOr(status, ADACODE_STATUS_ESCAPE_UNDERRUN);
                ++rank;
                row16[el] = (uint16_t)((row16[el] & 0x807Fu) | (e << 7));
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void decode_dispatch(AttnSmem &s, const adacode_segment &sg, int bh, int D, int which,
                                                int32_t *status) {
    if (s.lut_nbits[which] != sg.nbits || s.lut_left[which] != sg.left) {
        __syncthreads();
        build_decode_lut(s.lut[which], sg.nbits, sg.left, kAttnThreads);
        if (threadIdx.x == 0) {
            s.lut_nbits[which] = sg.nbits;
            s.lut_left[which] = sg.left;
        }
        __syncthreads();
    }
    switch (sg.nbits) {
        case 1: decode_tile<1>(s, sg, bh, D, s.lut[which], status); break;
        case 2: decode_tile<2>(s, sg, bh, D, s.lut[which], status); break;
        case 3: decode_tile<3>(s, sg, bh, D, s.lut[which], status); break;
        default: decode_tile<4>(s, sg, bh, D, s.lut[which], status); break;
    }
}

// Dense tile from the residual: rows [t0, t0 + 128) of `base`, zero beyond `len`.
__device__ __forceinline__ void load_dense_tile(AttnSmem &s, const uint16_t *base, long long ss, int t0, int len, int D) {
    const int row_stride = D + 2;
    const int words_per_row = D / 2;
    for (int i = threadIdx.x; i < kTileTokens * words_per_row; i += kAttnThreads) {
        const int row = i / words_per_row, w = i - row * words_per_row;
        uint32_t v = 0;
        if (t0 + row < len) v = *reinterpret_cast<const uint32_t *>(base + (long long)(t0 + row) * ss + 2 * w);
        *reinterpret_cast<uint32_t *>(s.tile + row * row_stride + 2 * w) = v;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kAttnThreads) k_decode_attn(const AttnArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttnSmem &s = *reinterpret_cast<AttnSmem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bh = blockIdx.x, split = blockIdx.y;      // (batch, KV head) on x: no 65 535 limit
    const int b = bh / a.Hkv, hkv = bh - b * a.Hkv;
    // query heads of the group are handled eight at a time: blockIdx.z picks the eight
    const int Gt = a.G, gz = blockIdx.z * kMaxGroup;
    const int G = Gt - gz < kMaxGroup ? Gt - gz : kMaxGroup, D = a.D;

    // queries of this KV head's group, as fp32, pre-multiplied by the softmax scale
    for (int i = tid; i < G * D; i += kAttnThreads) {
        const int g = i / D, d = i - g * D;
        const uint16_t raw = a.q[(long long)b * a.q_sb + (long long)(hkv * Gt + gz + g) * a.q_sh + d];
        s.q[g][d] = __uint_as_float((uint32_t)raw << 16) * a.scale;
    }
    for (int i = tid; i < kTileTokens * kMaxGroup; i += kAttnThreads) (&s.p[0][0])[i] = 0.f;
    if (tid == 0) s.lut_nbits[0] = s.lut_nbits[1] = 0;
    __syncthreads();

    const int tail_tiles = (a.tail_len + kTileTokens - 1) / kTileTokens;
    const int items = a.n_seg + tail_tiles;
    const int first = (int)((long long)items * split / a.n_splits);
    const int last = (int)((long long)items * (split + 1) / a.n_splits);

    float m[kMaxGroup], l[kMaxGroup], o[kMaxGroup];     // o: column `tid` of the numerator
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) m[g] = -INFINITY, l[g] = 0.f, o[g] = 0.f;
    const int row_words = (D + 2) / 2;

    for (int it = first; it < last; ++it) {
        const bool packed = it < a.n_seg;
        const int t0 = packed ? 0 : (it - a.n_seg) * kTileTokens;
        const int valid = packed ? kTileTokens : min(kTileTokens, a.tail_len - t0);
        // ---- K tile -> scores
        if (packed) decode_dispatch(s, a.kseg[it], bh, D, 0, a.status);
        else load_dense_tile(s, a.k_tail + (long long)b * a.t_sb + (long long)hkv * a.t_sh, a.t_ss, t0, a.tail_len, D);
        float sc[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) sc[g] = 0.f;
        const uint32_t *krow = reinterpret_cast<const uint32_t *>(s.tile) + tid * row_words;
        for (int j = 0; j < D / 2; ++j) {
            const uint32_t kw = krow[j];
            const float k0 = bf16_lo(kw), k1 = bf16_hi(kw);
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g)
                if (g < G) sc[g] = fmaf(s.q[g][2 * j], k0, fmaf(s.q[g][2 * j + 1], k1, sc[g]));
        }
        // ---- online softmax over the tile's 128 tokens (thread = token)
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                float v = tid < valid ? sc[g] : -INFINITY;
                sc[g] = v;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, d));
                if (lane == 0) s.red[g][warp] = v;
            }
        }
        __syncthreads();
        float alpha[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            alpha[g] = 1.f;
            if (g < G) {
                const float tmax = fmaxf(fmaxf(s.red[g][0], s.red[g][1]), fmaxf(s.red[g][2], s.red[g][3]));
                const float mn = fmaxf(m[g], tmax);
                alpha[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn);
                const float pv = (sc[g] == -INFINITY) ? 0.f : __expf(sc[g] - mn);
                s.p[tid][g] = pv;
                m[g] = mn;
                sc[g] = pv;
            }
        }
        __syncthreads();          // s.red is read, s.p is written
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                float v = sc[g];
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(kFull, v, d);
                if (lane == 0) s.red[g][warp] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g)
            if (g < G) l[g] = l[g] * alpha[g] + (s.red[g][0] + s.red[g][1] + s.red[g][2] + s.red[g][3]);
        // ---- V tile -> numerator (thread = output column)
        __syncthreads();          // everyone is done with the K tile and s.red
        if (packed) decode_dispatch(s, a.vseg[it], bh, D, 1, a.status);
        else load_dense_tile(s, a.v_tail + (long long)b * a.t_sb + (long long)hkv * a.t_sh, a.t_ss, t0, a.tail_len, D);
        if (tid < D) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) o[g] *= alpha[g];
            for (int t = 0; t < valid; ++t) {
                const float v = __uint_as_float((uint32_t)s.tile[t * (D + 2) + tid] << 16);
                const float4 p0 = *reinterpret_cast<const float4 *>(&s.p[t][0]);
                const float4 p1 = *reinterpret_cast<const float4 *>(&s.p[t][4]);
                o[0] = fmaf(p0.x, v, o[0]), o[1] = fmaf(p0.y, v, o[1]), o[2] = fmaf(p0.z, v, o[2]), o[3] = fmaf(p0.w, v, o[3]);
                o[4] = fmaf(p1.x, v, o[4]), o[5] = fmaf(p1.y, v, o[5]), o[6] = fmaf(p1.z, v, o[6]), o[7] = fmaf(p1.w, v, o[7]);
            }
        }
        __syncthreads();          // the tile and s.p are reused by the next item
    }

    const long long slot = (long long)bh * a.n_splits + split;
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) {
        if (g < G) {
            if (tid < D) a.part_o[(slot * Gt + gz + g) * D + tid] = o[g];
            if (tid == g) {
                a.part_ml[(slot * Gt + gz + g) * 2 + 0] = m[g];
                a.part_ml[(slot * Gt + gz + g) * 2 + 1] = l[g];
            }
        }
    }
}

// out[b][hq][d] = sum_s w_s o_s / sum_s w_s l_s, w_s = exp(m_s - max m)
__global__ void k_decode_attn_combine(const float *__restrict__ part_o, const float *__restrict__ part_ml, int Hq,
                                      int Hkv, int G, int D, int n_splits, uint16_t *__restrict__ out) {
    const int bhq = blockIdx.x;
    const int b = bhq / Hq, hq = bhq - b * Hq;
    const int hkv = hq / G, g = hq - hkv * G;
    const int d = threadIdx.x;
    if (d >= D) return;
    // launched as a programmatic dependent of the attention kernel: wait for its partial results
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long base = ((long long)b * Hkv + hkv) * n_splits;
    float mx = -INFINITY;
    for (int sidx = 0; sidx < n_splits; ++sidx) mx = fmaxf(mx, part_ml[((base + sidx) * G + g) * 2]);
    float num = 0.f, den = 0.f;
    for (int sidx = 0; sidx < n_splits; ++sidx) {
        const float ms = part_ml[((base + sidx) * G + g) * 2];
        if (ms == -INFINITY) continue;
        const float w = __expf(ms - mx);
        num = fmaf(w, part_o[((base + sidx) * G + g) * D + d], num);
        den = fmaf(w, part_ml[((base + sidx) * G + g) * 2 + 1], den);
    }
    const float r = den > 0.f ? num / den : 0.f;
    // round to nearest even bf16
    uint32_t u = __float_as_uint(r);
    u += 0x7FFFu + ((u >> 16) & 1u);
    out[(long long)bhq * D + d] = (uint16_t)(u >> 16);
}

// =======================================================================================
// Pipelined variant for head_dim 128: the unpack pipeline (producer warp, bulk copies into a
// two-stage ring, 16 consumer warps decoding out of shared memory) feeding tensor-core products.
// A decoded tile lives in shared memory as 128 rows (tokens) of 256 bytes whose 16-byte pieces are
// XOR-swizzled with the row index, so that ldmatrix reads it with few bank conflicts both as
// K (token-major, for scores) and, transposed, as V (for the weighted sum).
//   scores  S[t][g]   = sum_d K[t][d] q[g][d]   : mma.m16n8k16, A = K rows, B = q (8 query heads)
//   output  O^T[d][g] = sum_t V[t][d] P[t][g]   : mma.m16n8k16, A = V^T (ldmatrix.trans), B = P
// Warps 0..7 own 16 tokens (scores) resp. 16 output columns (weighted sum) each.
// =======================================================================================

constexpr int kAD = 128;                 // head_dim of this variant
constexpr int kQPad = kAD + 8;           // padded rows of the small operand matrices (272 bytes)
constexpr float kLog2e = 1.4426950408889634f;

struct AttnPipeSmem {
    UnpackStage stage[kStages];
    alignas(128) uint8_t tile[kTileTokens * kAD * 2];
    alignas(16) uint32_t lut[2][1024];            // [0] keys, [1] values
    alignas(16) uint16_t q[kMaxGroup][kQPad];     // queries, bf16
    alignas(16) uint16_t p[kMaxGroup][kQPad];     // probabilities of the current tile, bf16, [head][token]
    float red_max[8][kMaxGroup];                  // per-warp partial maxima
    float red_sum[8][kMaxGroup];                  // per-warp partial sums
    float m[2][kMaxGroup];                        // running max (log2 domain), double-buffered by tile parity
    float l[kMaxGroup];
    float alpha[kMaxGroup];
    alignas(8) uint64_t full[kStages];
    alignas(8) uint64_t empty[kStages];
    int warp_tot[kPWarps];
};

// Byte offset of 16-byte piece `piece` of row `row` in the swizzled tile.  Only the two low bits of
// the row enter the XOR: ldmatrix then sees two-way conflicts (eight rows, four patterns), which
// hardly matters at sixteen ldmatrix per warp and tile, and in return rows r and r + 4 share one
// pattern, so the second chunk of a thread (32 chunks = 4 rows further on) lies exactly 1024 bytes
// after the first and the second piece of a chunk at its first piece's offset XOR 16.
__device__ __forceinline__ uint32_t swz(int row, int piece) {
    return (uint32_t)(row * 256 + ((piece ^ (row & 3)) << 4));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
    uint32_t u = __float_as_uint(x);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return u >> 16;
}

// Decode one staged unit (a whole 128 x 128 tile) into the swizzled tile.  Same steps as the
// unpack kernel's consumer: zero-slot masks, warp scan, cross-warp prefix (one barrier), table
// decode, escapes OR-ed in.  Ends with a consumer barrier: the tile is complete on return.
template <int N>
__device__ __forceinline__ void decode_unit_swz(AttnPipeSmem &s, const UnpackStage &st, uint64_t *empty_bar,
                                                const uint32_t *lut, int32_t *status) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const UnitMeta m = st.meta;
    const int chunks = m.elems >> 4;

    uint4 o[kPCPT][2];
    uint32_t zm[kPCPT][2];
    int zc[kPCPT];
    decode_chunks<N>(st, lut, chunks, o, zm, zc);
    int incl[kPCPT];
    const int wtot = warp_scan_counts(zc, incl);
    if (lane == 0) s.warp_tot[warp] = wtot;
    consumer_sync();           // also: every warp is done reading the previous tile
    int wprefix, unit_tot;
    cross_warp_prefix(s.warp_tot, wprefix, unit_tot);
    static_assert(kPCPT == 2, "the escape loop below walks the two chunks of a thread together");
    const int c0 = warp * (kPCPT * 32) + lane;
    const uint32_t off0 = swz(c0 >> 3, (c0 & 7) * 2);          // chunk 0, first piece
    uint32_t *tile32 = reinterpret_cast<uint32_t *>(s.tile);
#pragma unroll
    for (int k = 0; k < kPCPT; ++k) {
        if (c0 + k * 32 < chunks) {
            *reinterpret_cast<uint4 *>(s.tile + off0 + 1024 * k) = o[k][0];
            *reinterpret_cast<uint4 *>(s.tile + (off0 ^ 16u) + 1024 * k) = o[k][1];
        }
    }
    if (zc[0] + zc[1] != 0) {
        const int r0 = wprefix + incl[0] - zc[0], r1 = wprefix + incl[1] - zc[1];     // ranks inside the tile
        const bool staged = (zc[0] == 0 || r0 + zc[0] <= m.esc_staged) && (zc[1] == 0 || r1 + zc[1] <= m.esc_staged);
        const uint32_t base_w = off0 >> 2;
        if (staged) {
            // one loop over the escapes of both chunks, as in the unpack kernel: chunk 0 elements
            // 0..15, then chunk 1 elements 0..15, from the most significant bit of the mask
            uint32_t todo = (compress_slots<N>(zm[0][0]) << 24) | (compress_slots<N>(zm[0][1]) << 16) |
                            (compress_slots<N>(zm[1][0]) << 8) | compress_slots<N>(zm[1][1]);
            const uint8_t *ep = st.esc + m.esc_shift + r0;
            const int skip = r1 - r0 - zc[0];
            int n = 0;
            while (todo) {
                const int i = __clz(todo);
                todo &= ~(0x80000000u >> i);
                const uint32_t e = ep[n + (i >> 4) * skip];
                ++n;
                const uint32_t t = (uint32_t)i >> 1;         // bit 2: second piece; bits 0..1: word in the piece
                atomicOr(tile32 + ((base_w ^ (t & 4u)) + (((uint32_t)i >> 4) << 8) + (t & 3u)), e << (7 + 16 * (i & 1)));
            }
        } else {
            // beyond the staged window (or beyond the stream): fetch from global memory
#pragma unroll 1
            for (int k = 0; k < kPCPT; ++k) {
                int r = k == 0 ? r0 : r1;
#pragma unroll 1
                for (int q = 0; q < 2; ++q) {
                    uint32_t z = k == 0 ? (q == 0 ? zm[0][0] : zm[0][1]) : (q == 0 ? zm[1][0] : zm[1][1]);
                    uint32_t *w32 = tile32 + ((base_w ^ ((uint32_t)q << 2)) + ((uint32_t)k << 8));
                    while (z) {
                        const int pos = 31 - __clz(z);
                        z ^= 1u << pos;
                        const int el = 7 - pos / N;
                        uint32_t e = 0;
                        if (r < m.esc_staged) e = st.esc[m.esc_shift + r];
                        else if (m.esc_tile_start + r < m.esc_len) e = m.esc[m.esc_tile_start + r];
                        else atomicOr(status, ADACODE_STATUS_ESCAPE_UNDERRUN);
                        ++r;
                        atomicOr(w32 + (el >> 1), e << (7 + 16 * (el & 1)));
                    }
                }
            }
        }
    }
    mbar_arrive(empty_bar);
    consumer_sync();
}

// Dense rows [t0, t0 + 128) of `base` into the swizzled tile, zero beyond `len`.  Barrier before
// (the previous tile is no longer read) and after (the tile is complete).
__device__ __forceinline__ void load_dense_tile_swz(AttnPipeSmem &s, const uint16_t *base, long long ss, int t0, int len) {
    consumer_sync();
    for (int i = threadIdx.x; i < kTileTokens * (kAD / 2); i += kConsumerThreads) {
        const int row = i >> 6, w = i & 63;
        uint32_t v = 0;
        if (t0 + row < len) v = *reinterpret_cast<const uint32_t *>(base + (long long)(t0 + row) * ss + 2 * w);
        *reinterpret_cast<uint32_t *>(s.tile + swz(row, w >> 2) + (w & 3) * 4) = v;
    }
    consumer_sync();
}

struct AttnPipeArgs {
    AttnArgs a;
    UnpackPipeArgs k, v;      // table form, used through resolve_tile
};

// Scores of the K tile in shared memory against the group's queries, online-softmax bookkeeping
// and the tile's probabilities (bf16, s.p).  Called by all consumer warps; warps 0..7 work (and meet
// at a barrier of their own), the others go straight on to the next unit's register phase.
__device__ __forceinline__ void score_tile(AttnPipeSmem &s, int valid, float sc2, int parity) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g0 = 2 * (lane & 3), r0 = lane >> 2;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp < 8) {
        const uint32_t tile_base = smem_u32(s.tile);
        const int t0 = warp * 16;
        const int lrow = t0 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int lp = lane >> 4;
#pragma unroll
        for (int ks = 0; ks < kAD / 16; ++ks) {
            uint32_t af[4];
            ldsm_x4(tile_base + swz(lrow, 2 * ks + lp), af);
            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&s.q[r0][16 * ks + g0]);
            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(&s.q[r0][16 * ks + 8 + g0]);
            mma_bf16(c, af, b0, b1);
        }
        const int ta = t0 + r0, tb = ta + 8;
        c[0] = ta < valid ? c[0] * sc2 : -INFINITY;
        c[1] = ta < valid ? c[1] * sc2 : -INFINITY;
        c[2] = tb < valid ? c[2] * sc2 : -INFINITY;
        c[3] = tb < valid ? c[3] * sc2 : -INFINITY;
        float v0 = fmaxf(c[0], c[2]), v1 = fmaxf(c[1], c[3]);
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
            v0 = fmaxf(v0, __shfl_xor_sync(kFull, v0, d));
            v1 = fmaxf(v1, __shfl_xor_sync(kFull, v1, d));
        }
        if (lane < 4) {
            s.red_max[warp][g0] = v0;
            s.red_max[warp][g0 + 1] = v1;
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");      // the eight math warps only; the others run ahead
        float mn[2], al[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float tm = s.red_max[0][g0 + j];
#pragma unroll
            for (int w = 1; w < 8; ++w) tm = fmaxf(tm, s.red_max[w][g0 + j]);
            const float mo = s.m[parity][g0 + j];
            mn[j] = fmaxf(mo, tm);
            al[j] = mo == -INFINITY ? 0.f : exp2f(mo - mn[j]);
        }
        // probabilities, rounded to bf16 (what the tensor cores multiply with; the sums use the same)
        const uint32_t b00 = f32_to_bf16_bits(c[0] == -INFINITY ? 0.f : exp2f(c[0] - mn[0]));
        const uint32_t b01 = f32_to_bf16_bits(c[1] == -INFINITY ? 0.f : exp2f(c[1] - mn[1]));
        const uint32_t b10 = f32_to_bf16_bits(c[2] == -INFINITY ? 0.f : exp2f(c[2] - mn[0]));
        const uint32_t b11 = f32_to_bf16_bits(c[3] == -INFINITY ? 0.f : exp2f(c[3] - mn[1]));
        s.p[g0][ta] = (uint16_t)b00;
        s.p[g0 + 1][ta] = (uint16_t)b01;
        s.p[g0][ta + 8] = (uint16_t)b10;
        s.p[g0 + 1][ta + 8] = (uint16_t)b11;
        float s0 = __uint_as_float(b00 << 16) + __uint_as_float(b10 << 16);
        float s1 = __uint_as_float(b01 << 16) + __uint_as_float(b11 << 16);
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
            s0 += __shfl_xor_sync(kFull, s0, d);
            s1 += __shfl_xor_sync(kFull, s1, d);
        }
        if (lane < 4) {
            s.red_sum[warp][g0] = s0;
            s.red_sum[warp][g0 + 1] = s1;
            if (warp == 0) {
                s.m[parity ^ 1][g0] = mn[0];
                s.m[parity ^ 1][g0 + 1] = mn[1];
                s.alpha[g0] = al[0];
                s.alpha[g0 + 1] = al[1];
            }
        }
    }
}

// oacc = oacc * alpha + V^T P for the V tile in shared memory; warp 0 also folds the tile's
// probability sums into the running denominators.  The caller has passed a barrier since score_tile.
__device__ __forceinline__ void accumulate_tile(AttnPipeSmem &s, float (&oacc)[4]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g0 = 2 * (lane & 3), r0 = lane >> 2;
    if (warp >= 8) return;
    const float a0 = s.alpha[g0], a1 = s.alpha[g0 + 1];
    oacc[0] *= a0, oacc[1] *= a1, oacc[2] *= a0, oacc[3] *= a1;
    const uint32_t tile_base = smem_u32(s.tile);
    const int m_piece = warp * 2 + ((lane >> 3) & 1);            // output columns 16 warp .. 16 warp + 15
    const int lt = (lane & 7) + (lane >> 4) * 8;
#pragma unroll
    for (int ks = 0; ks < kTileTokens / 16; ++ks) {
        uint32_t af[4];
        ldsm_x4_trans(tile_base + swz(16 * ks + lt, m_piece), af);
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&s.p[r0][16 * ks + g0]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t *>(&s.p[r0][16 * ks + 8 + g0]);
        mma_bf16(oacc, af, b0, b1);
    }
    if (warp == 0 && lane < kMaxGroup) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += s.red_sum[w][lane];
        s.l[lane] = s.l[lane] * s.alpha[lane] + t;
    }
}

__global__ void __launch_bounds__(kPipeThreads, 2) k_decode_attn_pipe(const AttnPipeArgs pa) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttnPipeSmem &s = *reinterpret_cast<AttnPipeSmem *>(smem_raw);
    const AttnArgs &a = pa.a;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bh = blockIdx.x, split = blockIdx.y;      // (batch, KV head) on x: no 65 535 limit
    const int b = bh / a.Hkv, hkv = bh - b * a.Hkv;
    const int Gt = a.G, gz = blockIdx.z * kMaxGroup;     // eight query heads of the group per CTA
    const int G = Gt - gz < kMaxGroup ? Gt - gz : kMaxGroup;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], kConsumerThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // launched as a programmatic dependent of its predecessor in the stream: no global memory is touched above
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // queries (zero rows beyond G), running statistics
    for (int i = tid; i < kMaxGroup * kQPad; i += kPipeThreads) {
        const int g = i / kQPad, d = i - g * kQPad;
        uint16_t v = 0;
        if (g < G && d < kAD) v = a.q[(long long)b * a.q_sb + (long long)(hkv * Gt + gz + g) * a.q_sh + d];
        s.q[g][d] = v;
        s.p[g][d] = 0;
    }
    if (tid < kMaxGroup) {
        s.m[0][tid] = s.m[1][tid] = -INFINITY;
        s.l[tid] = 0.f;
        s.alpha[tid] = 0.f;
    }
    __syncthreads();

    const int tail_tiles = (a.tail_len + kTileTokens - 1) / kTileTokens;
    const int items = a.n_seg + tail_tiles;
    const int first = (int)((long long)items * split / a.n_splits);
    const int last = (int)((long long)items * (split + 1) / a.n_splits);
    const int pk_first = first < a.n_seg ? first : a.n_seg;
    const int pk_last = last < a.n_seg ? last : a.n_seg;
    const int n_units = 2 * (pk_last - pk_first);          // K tile, V tile, K tile, ...

    if (tid >= kConsumerThreads) {
        // ---------------- producer warp ----------------
        uint32_t it = 0;
        for (int base = 0; base < n_units; base += 32) {
            TileSrc mine = {};
            const int u = base + lane;
            if (u < n_units) {
                const long long tile = (long long)(pk_first + (u >> 1)) * pa.k.BH + bh;
                mine = (u & 1) ? resolve_tile(pa.v, tile) : resolve_tile(pa.k, tile);
            }
            const int n_here = n_units - base < 32 ? n_units - base : 32;
            for (int j = 0; j < n_here; ++j, ++it) {
                const TileSrc t = shfl_tile(mine, j);
                const EscWindow w = esc_window(t);
                const int stg = it % kStages;
                mbar_wait(&s.empty[stg], ((it / kStages) & 1) ^ 1, a.status);
                issue_unit(s.stage[stg], s.stage[stg].meta, &s.full[stg], t, w, 0, kTileTokens, kAD, nullptr, true, a.status);
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const float sc2 = a.scale * kLog2e;                      // scores are kept in the log2 domain
    float oacc[4] = {0.f, 0.f, 0.f, 0.f};                    // O^T[d = 16 warp + lane/4 (+8)][2 (lane%4), +1]
    int parity = 0;                                          // tiles seen & 1: which m[] holds the running max
    int lut_left[2] = {0, 0}, lut_nbits[2] = {0, 0};
    for (int u = 0; u < n_units; ++u) {
        const int stg = u % kStages, which = u & 1;
        if (lane == 0) mbar_wait(&s.full[stg], (u / kStages) & 1, a.status);
        __syncwarp();
        const UnpackStage &st = s.stage[stg];
        const int nb = st.meta.nbits, lf = st.meta.left;
        if (nb != lut_nbits[which] || lf != lut_left[which]) {
            // uniform over the CTA; the previous user of this table finished before the last barrier
            build_decode_lut(s.lut[which], nb, lf, kConsumerThreads);
            lut_nbits[which] = nb, lut_left[which] = lf;
            consumer_sync();
        }
        switch (nb) {
            case 1: decode_unit_swz<1>(s, st, &s.empty[stg], s.lut[which], a.status); break;
            case 2: decode_unit_swz<2>(s, st, &s.empty[stg], s.lut[which], a.status); break;
            case 3: decode_unit_swz<3>(s, st, &s.empty[stg], s.lut[which], a.status); break;
            default: decode_unit_swz<4>(s, st, &s.empty[stg], s.lut[which], a.status); break;
        }
        if (which == 0) {
            score_tile(s, kTileTokens, sc2, parity);
        } else {
            accumulate_tile(s, oacc);
            parity ^= 1;
        }
    }
    // dense residual tiles that fall into this split
    const int tl_first = first > a.n_seg ? first - a.n_seg : 0;
    const int tl_last = last > a.n_seg ? last - a.n_seg : 0;
    for (int j = tl_first; j < tl_last; ++j) {
        const int t0 = j * kTileTokens;
        const int valid = a.tail_len - t0 < kTileTokens ? a.tail_len - t0 : kTileTokens;
        const long long off = (long long)b * a.t_sb + (long long)hkv * a.t_sh;
        load_dense_tile_swz(s, a.k_tail + off, a.t_ss, t0, a.tail_len);
        score_tile(s, valid, sc2, parity);
        load_dense_tile_swz(s, a.v_tail + off, a.t_ss, t0, a.tail_len);
        accumulate_tile(s, oacc);
        parity ^= 1;
    }
    consumer_sync();
    const long long slot = (long long)bh * a.n_splits + split;
    if (warp < 8) {
        const int g0 = 2 * (lane & 3), d0 = warp * 16 + (lane >> 2);
        if (g0 < G) {
            a.part_o[(slot * Gt + gz + g0) * kAD + d0] = oacc[0];
            a.part_o[(slot * Gt + gz + g0) * kAD + d0 + 8] = oacc[2];
        }
        if (g0 + 1 < G) {
            a.part_o[(slot * Gt + gz + g0 + 1) * kAD + d0] = oacc[1];
            a.part_o[(slot * Gt + gz + g0 + 1) * kAD + d0 + 8] = oacc[3];
        }
    }
    if (tid < G) {
        const float m2 = s.m[parity][tid];
        a.part_ml[(slot * Gt + gz + tid) * 2 + 0] = m2 == -INFINITY ? -INFINITY : m2 / kLog2e;   // natural-log domain
        a.part_ml[(slot * Gt + gz + tid) * 2 + 1] = s.l[tid];
    }
}

static_assert(sizeof(AttnPipeSmem) <= 113 * 1024, "two CTAs of the pipelined kernel must fit one SM");

constexpr int kMaxSplits = 128;

// Splits per (batch, KV head): the grid should fill a whole number of waves of resident CTAs
// (two per SM for the pipelined kernel, three for the plain one).  One, two and three waves are
// tried and the fullest wins; fewer waves on ties (more tiles per CTA, less per-CTA overhead).
int pick_splits(int B, int Hkv, int items, int D) {
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long slots = (long long)sms * (D == kAD ? 2 : 3);
    const long long bh = (long long)B * Hkv;
    int best = 1;
    double best_fill = 0.0;
    for (int waves = 1; waves <= 3; ++waves) {
        long long sp = waves * slots / bh;
        if (sp < 1) sp = 1;
        if (sp > items) sp = items;
        if (sp > kMaxSplits) sp = kMaxSplits;
        const long long ctas = bh * sp;
        const double fill = (double)ctas / (double)(((ctas + slots - 1) / slots) * slots);
        if (fill > best_fill + 0.02) best_fill = fill, best = (int)sp;
    }
    return best;
}

}  // namespace

namespace {
// Programmatic dependent launch: the kernel may be set up while its predecessor in the stream drains;
// it executes griddepcontrol.wait before it reads or writes global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_as_dependent(void (*kernel)(KArgs...), dim3 grid, int threads, size_t smem, cudaStream_t st,
                                Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = dim3(threads), cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace

extern "C" {

size_t adacode_decode_attn_workspace_bytes(int B, int Hq, int D, int n_splits) {
    if (B <= 0 || Hq <= 0 || D <= 0) return 0;
    if (n_splits <= 0 || n_splits > kMaxSplits) n_splits = kMaxSplits;
    return (size_t)B * Hq * n_splits * ((size_t)D + 2) * sizeof(float);
}

int adacode_decode_attn(const void *q_bf16, int64_t q_stride_b, int64_t q_stride_h,
                        const adacode_segment *k_segments_dev, const adacode_segment *v_segments_dev, int n_segments,
                        const void *k_tail_bf16, const void *v_tail_bf16, int tail_len, int64_t tail_stride_b,
                        int64_t tail_stride_h, int64_t tail_stride_s, int B, int Hq, int Hkv, int seq_tile, int D,
                        float scale, void *out_bf16, void *workspace, size_t workspace_bytes, int n_splits,
                        int32_t *status, void *stream) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || n_segments < 0 || tail_len < 0) return ADACODE_ERR_INVALID_ARG;
    const int G = Hq / Hkv;
    if (seq_tile != kTileTokens || (D != 64 && D != 128)) return ADACODE_ERR_INVALID_ARG;
    const int head_groups = (G + kMaxGroup - 1) / kMaxGroup;      // CTAs along z, eight query heads each
    if (head_groups > 65535) return ADACODE_ERR_INVALID_ARG;
    if (!q_bf16 || !out_bf16 || !workspace || !status) return ADACODE_ERR_INVALID_ARG;
    if (n_segments > 0 && (!k_segments_dev || !v_segments_dev)) return ADACODE_ERR_INVALID_ARG;
    if (tail_len > 0 && (!k_tail_bf16 || !v_tail_bf16 || ((uintptr_t)k_tail_bf16 & 3) || ((uintptr_t)v_tail_bf16 & 3) ||
                         ((tail_stride_b | tail_stride_h | tail_stride_s) & 1)))
        return ADACODE_ERR_INVALID_ARG;
    const int items = n_segments + (tail_len + kTileTokens - 1) / kTileTokens;
    if (items == 0) return ADACODE_ERR_INVALID_ARG;
    if (n_splits <= 0) n_splits = pick_splits(B, Hkv * head_groups, items, D);
    if (n_splits > kMaxSplits) n_splits = kMaxSplits;
    if (workspace_bytes < adacode_decode_attn_workspace_bytes(B, Hq, D, n_splits)) return ADACODE_ERR_WORKSPACE;
    AttnArgs a;
    a.q = (const uint16_t *)q_bf16, a.q_sb = q_stride_b, a.q_sh = q_stride_h;
    a.kseg = k_segments_dev, a.vseg = v_segments_dev, a.n_seg = n_segments;
    a.k_tail = (const uint16_t *)k_tail_bf16, a.v_tail = (const uint16_t *)v_tail_bf16, a.tail_len = tail_len;
    a.t_sb = tail_stride_b, a.t_sh = tail_stride_h, a.t_ss = tail_stride_s;
    a.B = B, a.Hq = Hq, a.Hkv = Hkv, a.G = G, a.D = D, a.scale = scale, a.n_splits = n_splits;
    a.part_o = (float *)workspace;
    a.part_ml = a.part_o + (size_t)B * Hq * n_splits * D;
    a.status = status;
    cudaStream_t st = (cudaStream_t)stream;
    static bool attr_set[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return ADACODE_ERR_CUDA;
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(k_decode_attn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnSmem)) !=
                cudaSuccess ||
            cudaFuncSetAttribute(k_decode_attn_pipe, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)sizeof(AttnPipeSmem)) != cudaSuccess)
            return ADACODE_ERR_CUDA;
        attr_set[dev] = true;
    }
    // head_dim 128: the pipelined tensor-core kernel; ADACODE_ATTN_SIMPLE=1 forces the plain one
    static const bool force_simple = [] {
        const char *v = getenv("ADACODE_ATTN_SIMPLE");
        return v && v[0] == '1';
    }();
    if (D == kAD && !force_simple) {
        AttnPipeArgs pa;
        pa.a = a;
        UnpackPipeArgs u;
        u.sign_mant = nullptr, u.codes = nullptr, u.escapes = nullptr, u.escapes_len = 0;
        u.tile_base = nullptr, u.seg_off = nullptr, u.left = 0, u.nbits = 0;
        u.tb_stride = 1, u.tb_before = 0;
        u.H = Hkv, u.BH = B * Hkv, u.seq_tile = kTileTokens, u.D = D, u.tile_elems = kTileTokens * D;
        u.n_tiles = (long long)n_segments * B * Hkv;
        u.dst = nullptr, u.db = 0, u.dh = 0, u.ds = 0, u.status = status;
        pa.k = u, pa.v = u;
        pa.k.seg = k_segments_dev, pa.v.seg = v_segments_dev;
        if (launch_as_dependent(k_decode_attn_pipe, dim3(B * Hkv, n_splits, head_groups), kPipeThreads,
                                sizeof(AttnPipeSmem), st, pa) != cudaSuccess)
            return ADACODE_ERR_CUDA;
    } else {
        k_decode_attn<<<dim3(B * Hkv, n_splits, head_groups), kAttnThreads, sizeof(AttnSmem), st>>>(a);
    }
    if (cudaGetLastError() != cudaSuccess) return ADACODE_ERR_CUDA;
    if (launch_as_dependent(k_decode_attn_combine, dim3(B * Hq), D, 0, st, (const float *)a.part_o,
                            (const float *)a.part_ml, Hq, Hkv, G, D, n_splits, (uint16_t *)out_bf16) != cudaSuccess)
        return ADACODE_ERR_CUDA;
    return ADACODE_OK;
}

}  // extern "C"
