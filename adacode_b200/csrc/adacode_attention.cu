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

namespace {

#include "adacode_device.cuh"

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
    extern __shared__ __align__(16) uint8_t smem_raw[];
    AttnSmem &s = *reinterpret_cast<AttnSmem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, bh = blockIdx.y;
    const int b = bh / a.Hkv, hkv = bh - b * a.Hkv;
    const int G = a.G, D = a.D;

    // queries of this KV head's group, as fp32, pre-multiplied by the softmax scale
    for (int i = tid; i < G * D; i += kAttnThreads) {
        const int g = i / D, d = i - g * D;
        const uint16_t raw = a.q[(long long)b * a.q_sb + (long long)(hkv * G + g) * a.q_sh + d];
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
            if (tid < D) a.part_o[(slot * G + g) * D + tid] = o[g];
            if (tid == g) {
                a.part_ml[(slot * G + g) * 2 + 0] = m[g];
                a.part_ml[(slot * G + g) * 2 + 1] = l[g];
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

int pick_splits(int B, int Hkv, int items) {
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int want = (3 * sms + B * Hkv - 1) / (B * Hkv);     // about three CTAs per SM
    if (want > items) want = items;
    if (want < 1) want = 1;
    if (want > 64) want = 64;
    return want;
}

}  // namespace

extern "C" {

size_t adacode_decode_attn_workspace_bytes(int B, int Hq, int D, int n_splits) {
    if (B <= 0 || Hq <= 0 || D <= 0) return 0;
    if (n_splits <= 0) n_splits = 64;
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
    if (G > kMaxGroup || seq_tile != kTileTokens || (D != 64 && D != 128)) return ADACODE_ERR_INVALID_ARG;
    if (!q_bf16 || !out_bf16 || !workspace || !status) return ADACODE_ERR_INVALID_ARG;
    if (n_segments > 0 && (!k_segments_dev || !v_segments_dev)) return ADACODE_ERR_INVALID_ARG;
    if (tail_len > 0 && (!k_tail_bf16 || !v_tail_bf16 || ((uintptr_t)k_tail_bf16 & 3) || ((uintptr_t)v_tail_bf16 & 3) ||
                         ((tail_stride_b | tail_stride_h | tail_stride_s) & 1)))
        return ADACODE_ERR_INVALID_ARG;
    const int items = n_segments + (tail_len + kTileTokens - 1) / kTileTokens;
    if (items == 0) return ADACODE_ERR_INVALID_ARG;
    if (n_splits <= 0) n_splits = pick_splits(B, Hkv, items);
    if (n_splits > 64) n_splits = 64;
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
            cudaSuccess)
            return ADACODE_ERR_CUDA;
        attr_set[dev] = true;
    }
    k_decode_attn<<<dim3(n_splits, B * Hkv), kAttnThreads, sizeof(AttnSmem), st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return ADACODE_ERR_CUDA;
    k_decode_attn_combine<<<B * Hq, D, 0, st>>>(a.part_o, a.part_ml, Hq, Hkv, G, D, n_splits, (uint16_t *)out_bf16);
    if (cudaGetLastError() != cudaSuccess) return ADACODE_ERR_CUDA;
    return ADACODE_OK;
}

}  // extern "C"
