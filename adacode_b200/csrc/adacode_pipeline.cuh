// Pipelined pack / unpack kernels: tiles are staged through shared memory with asynchronous
// bulk copies (the untiled form of TMA) so that the loads of the next units are in flight
// while the current unit is processed, and results leave through shared memory with bulk
// stores.  Included by adacode_kernels.cu inside its anonymous namespace.
//
// One CTA = 8 consumer warps + 1 producer warp, persistent over tiles.  A "unit" is a run of
// whole token rows of one tile, at most 16384 elements (a whole 128 x 128 tile).
//   producer warp : waits for a free stage, issues the unit's bulk loads (sign/mantissa and
//                   code planes, or source rows) against the stage's "full" mbarrier, and
//                   stages the tile's escape bytes with plain loads
//   consumer warps: wait on "full", work out of shared memory, signal "empty", and hand the
//                   finished unit to a bulk store
// Every mbarrier wait is bounded: after kMaxPolls failed polls the waiter records
// ADACODE_STATUS_TIMEOUT in the status word and carries on (the result is then wrong but the
// kernel still reaches every barrier and terminates).
#pragma once

constexpr int kConsumerThreads = 256;
constexpr int kPipeThreads = kConsumerThreads + 32;
constexpr int kUnitElems = 16384;
constexpr int kStages = 2;
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; on expiry flags the status word and returns anyway.
__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity, int32_t *status) {
    for (uint32_t i = 0; i < kMaxPolls; ++i)
        if (mbar_try_wait(bar, parity)) return;
    atomicOr(status, ADACODE_STATUS_TIMEOUT);
}
// global -> shared bulk copy, completion counted in bytes on `bar`; 16-byte aligned, size % 16 == 0
__device__ __forceinline__ void bulk_load(void *sdst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(sdst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// shared -> global bulk copy, tracked by the issuing thread's bulk group
__device__ __forceinline__ void bulk_store(void *gdst, const void *ssrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// makes shared-memory writes of this thread visible to the async proxy (bulk stores)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Rows of one tile handled per unit: whole rows, a multiple of 8 (so that code bytes per unit are a
// multiple of 16), at most kUnitElems elements.
__host__ __device__ inline int unit_rows_for(int seq_tile, int D) {
    int r = (kUnitElems / D) & ~7;
    if (r < 8) r = 8;
    return r < seq_tile ? r : seq_tile;
}

// ---------------------------------------------------------------------------------------
// unpack
// ---------------------------------------------------------------------------------------

constexpr int kEscStage = 8192;   // bytes of a tile's escape stream staged in shared memory

struct UnitMeta {
    uint16_t *dst;            // first element of the unit in the destination
    const uint8_t *esc;       // the segment's escape stream
    long long esc_len;
    long long esc_tile_start; // index in esc of the tile's first escape
    int esc_staged;           // escapes of the tile present in shared memory (from index 0 of the tile)
    int esc_shift;            // offset of escape 0 inside the staged bytes
    int elems;
    int left;
    int nbits;
    int first_unit_of_tile;
};

// bulk copies need 16-byte aligned shared addresses: every buffer starts on a 128-byte boundary
struct alignas(128) UnpackStage {
    alignas(128) uint8_t sm[kUnitElems];
    alignas(128) uint8_t codes[kUnitElems / 2];
    alignas(128) uint8_t esc[kEscStage + 16];
    alignas(16) UnitMeta meta;
};

struct alignas(128) UnpackSmem {
    UnpackStage stage[kStages];
    alignas(128) uint16_t out[kUnitElems];
    alignas(8) uint64_t full[kStages];
    alignas(8) uint64_t empty[kStages];
    int warp_tot[kWarps];
};
static_assert(sizeof(UnpackStage) % 128 == 0, "stage buffers must stay 128-byte aligned");

struct UnpackPipeArgs {
    // uniform form (seg == nullptr): planes as adacode_pack_tiles wrote them
    const uint8_t *sign_mant;
    const uint8_t *codes;
    const uint8_t *escapes;
    long long escapes_len;
    const int32_t *tile_base;
    const int64_t *seg_off;
    int left, nbits;
    // table form
    const adacode_segment *seg;
    // common
    int H, BH, seq_tile, D, tile_elems;
    long long n_tiles;
    uint16_t *dst;
    long long db, dh, ds;
    int32_t *status;
};

// Everything the producer needs to know about tile `tile`.
struct TileSrc {
    const uint8_t *sm, *codes, *esc;
    long long esc_len, esc_start;
    int esc_cnt, left, nbits;
    uint16_t *dst;
};

__device__ __forceinline__ TileSrc resolve_tile(const UnpackPipeArgs &a, long long tile) {
    TileSrc t;
    const long long blk = tile / a.BH;
    const int bh = (int)(tile - blk * a.BH);
    const int b = bh / a.H, h = bh - b * a.H;
    uint16_t *base = a.dst + (long long)b * a.db + (long long)h * a.dh;
    if (a.seg) {
        const adacode_segment sg = a.seg[blk];
        t.nbits = sg.nbits, t.left = sg.left;
        t.sm = sg.sign_mant + (long long)bh * a.tile_elems;
        t.codes = sg.codes + (long long)bh * (a.tile_elems * sg.nbits / 8);
        t.esc = sg.escapes, t.esc_len = sg.escapes_len;
        const int prev = bh > 0 ? sg.tile_base[bh - 1] : 0;
        t.esc_start = prev;
        t.esc_cnt = sg.tile_base[bh] - prev;
        t.dst = base + sg.dst_seq_offset * a.ds;
    } else {
        t.nbits = a.nbits, t.left = a.left;
        t.sm = a.sign_mant + tile * a.tile_elems;
        t.codes = a.codes + tile * (a.tile_elems * a.nbits / 8);
        t.esc = a.escapes, t.esc_len = a.escapes_len;
        const long long seg_start = a.seg_off ? a.seg_off[blk] : 0;
        const int prev = bh > 0 ? a.tile_base[tile - 1] : 0;
        t.esc_start = seg_start + prev;
        t.esc_cnt = a.tile_base[tile] - prev;
        t.dst = base + blk * a.seq_tile * a.ds;
    }
    return t;
}

template <int N>
__device__ __forceinline__ void unpack_unit(UnpackSmem &s, const UnpackStage &st, uint64_t *empty_bar,
                                            long long &consumed, bool rows_contig, int D, long long ds,
                                            int32_t *status) {
    constexpr int CB = 2 * N;   // code bytes per 16-element chunk
    constexpr uint32_t kMask = (1u << N) - 1u;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const UnitMeta m = st.meta;
    if (m.first_unit_of_tile) consumed = 0;
    const int chunks = m.elems >> 4;
    const uint32_t left2 = ((uint32_t)m.left & 0xFFu) * 0x10001u;

    uint4 o[kCPT][2];
    uint32_t zm[kCPT][2];
    int zc[kCPT];
#pragma unroll
    for (int k = 0; k < kCPT; ++k) {
        const int c = warp * (kCPT * 32) + k * 32 + lane;
        uint32_t g[2] = {0u, 0u};
        uint4 sv = make_uint4(0, 0, 0, 0);
        const bool valid = c < chunks;
        if (valid) {
            sv = *reinterpret_cast<const uint4 *>(st.sm + c * 16);
            load_chunk_codes<N, 16>(st.codes + c * CB, g);
        }
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        zc[k] = 0;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            zm[k][q] = valid ? zero_slots<N>(g[q]) : 0u;
            zc[k] += __popc(zm[k][q]);
            uint32_t cd[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) cd[j] = (g[q] >> ((7 - j) * N)) & kMask;
            const uint32_t s0 = sw[2 * q], s1 = sw[2 * q + 1];
            o[k][q].x = assemble2(__byte_perm(s0, 0u, 0x4140), cd[0], cd[1], left2);
            o[k][q].y = assemble2(__byte_perm(s0, 0u, 0x4342), cd[2], cd[3], left2);
            o[k][q].z = assemble2(__byte_perm(s1, 0u, 0x4140), cd[4], cd[5], left2);
            o[k][q].w = assemble2(__byte_perm(s1, 0u, 0x4342), cd[6], cd[7], left2);
        }
    }
    int incl[kCPT];
    const int wtot = warp_scan4(zc, incl);
    if (lane == 0) s.warp_tot[warp] = wtot;
    bulk_wait_read();          // the previous unit's store has finished reading s.out
    consumer_sync();
    int wprefix = 0, unit_tot = 0;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) {
        const int t = s.warp_tot[i];
        wprefix += (i < warp) ? t : 0;
        unit_tot += t;
    }
#pragma unroll
    for (int k = 0; k < kCPT; ++k) {
        const int c = warp * (kCPT * 32) + k * 32 + lane;
        if (c < chunks) {
            uint4 *w = reinterpret_cast<uint4 *>(s.out + c * 16);
            w[0] = o[k][0];
            w[1] = o[k][1];
            if (zc[k] != 0) {
                long long r = consumed + wprefix + incl[k] - zc[k];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    uint32_t z = zm[k][q];
                    while (z) {
                        const int pos = 31 - __clz(z);
                        z ^= 1u << pos;
                        const int el = q * 8 + 7 - pos / N;
                        uint32_t e = 0;
                        if (r < m.esc_staged) {
                            e = st.esc[m.esc_shift + (int)r];
                        } else if (m.esc_tile_start + r < m.esc_len) {
                            e = m.esc[m.esc_tile_start + r];
                        } else {
                            atomicOr(status, ADACODE_STATUS_ESCAPE_UNDERRUN);
                        }
                        ++r;
                        uint16_t *pw = s.out + c * 16 + el;
                        *pw = (uint16_t)((*pw & 0x807Fu) | (e << 7));
                    }
                }
            }
        }
    }
    consumed += unit_tot;
    mbar_arrive(empty_bar);    // this thread no longer reads the stage
    fence_async_smem();
    consumer_sync();
    if (rows_contig) {
        if (tid == 0 && m.elems > 0) {
            bulk_store(m.dst, s.out, (uint32_t)m.elems * 2u);
            bulk_commit();
        }
    } else {
        const int rows = m.elems / D;
        for (int r = tid; r < rows; r += kConsumerThreads) bulk_store(m.dst + (long long)r * ds, s.out + r * D, (uint32_t)D * 2u);
        bulk_commit();
    }
}

__global__ void __launch_bounds__(kPipeThreads) k_unpack_pipe(const UnpackPipeArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    UnpackSmem &s = *reinterpret_cast<UnpackSmem *>(smem_raw);
    const int tid = threadIdx.x;
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], kConsumerThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int unit_rows = unit_rows_for(a.seq_tile, a.D);
    const int units_per_tile = (a.seq_tile + unit_rows - 1) / unit_rows;
    const bool rows_contig = (a.ds == a.D);

    if (tid >= kConsumerThreads) {
        // ---------------- producer warp ----------------
        const int lane = tid & 31;
        uint32_t it = 0;
        for (long long tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
            const TileSrc t = resolve_tile(a, tile);
            // stage no more than the stream really holds, so that a short stream is reported as such
            long long avail = t.esc_len - t.esc_start;
            if (avail > t.esc_cnt) avail = t.esc_cnt;
            if (avail > kEscStage) avail = kEscStage;
            const int staged = avail > 0 ? (int)avail : 0;
            const uint8_t *ea = t.esc + t.esc_start;
            const int shift = (int)((uintptr_t)ea & 15);
            for (int u = 0; u < units_per_tile; ++u, ++it) {
                const int stg = it % kStages;
                UnpackStage &st = s.stage[stg];
                mbar_wait(&s.empty[stg], ((it / kStages) & 1) ^ 1, a.status);
                // the tile's escape bytes (the same window for every unit of the tile)
                const uint8_t *a0 = ea - shift;
                const uint8_t *lo_ok = t.esc, *hi_ok = t.esc + t.esc_len;
                for (int wd = lane; wd * 16 < shift + staged; wd += 32) {
                    const uint8_t *p = a0 + wd * 16;
                    if (p >= lo_ok && p + 16 <= hi_ok) {
                        *reinterpret_cast<uint4 *>(st.esc + wd * 16) = __ldg(reinterpret_cast<const uint4 *>(p));
                    } else {
                        for (int b = 0; b < 16; ++b)
                            if (p + b >= lo_ok && p + b < hi_ok) st.esc[wd * 16 + b] = p[b];
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    const int row0 = u * unit_rows;
                    const int rows = min(unit_rows, a.seq_tile - row0);
                    const int elems = rows * a.D;
                    const uint8_t *src_sm = t.sm + (long long)row0 * a.D;
                    const uint8_t *src_cd = t.codes + (long long)row0 * a.D * t.nbits / 8;
                    UnitMeta &m = st.meta;
                    m.dst = t.dst + (long long)row0 * a.ds;
                    m.esc = t.esc, m.esc_len = t.esc_len, m.esc_tile_start = t.esc_start;
                    m.esc_staged = staged, m.esc_shift = shift;
                    m.elems = elems, m.left = t.left, m.nbits = t.nbits;
                    m.first_unit_of_tile = (u == 0);
                    const uint32_t cbytes = (uint32_t)elems * t.nbits / 8;
                    if ((((uintptr_t)src_sm | (uintptr_t)src_cd | (uintptr_t)m.dst) & 15) != 0 || (cbytes & 15) != 0 ||
                        t.nbits < 1 || t.nbits > 4) {
                        // never start a misaligned bulk copy: flag it and hand over an empty unit
                        atomicOr(a.status, ADACODE_STATUS_MISALIGNED);
                        m.elems = 0;
                        m.nbits = 1;
                        mbar_arrive_expect_tx(&s.full[stg], 0);
                    } else {
                        mbar_arrive_expect_tx(&s.full[stg], (uint32_t)elems + cbytes);
                        bulk_load(st.sm, src_sm, (uint32_t)elems, &s.full[stg]);
                        bulk_load(st.codes, src_cd, cbytes, &s.full[stg]);
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    uint32_t it = 0;
    long long consumed = 0;
    for (long long tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
        for (int u = 0; u < units_per_tile; ++u, ++it) {
            const int stg = it % kStages;
            mbar_wait(&s.full[stg], (it / kStages) & 1, a.status);
            const UnpackStage &st = s.stage[stg];
            switch (st.meta.nbits) {
                case 1: unpack_unit<1>(s, st, &s.empty[stg], consumed, rows_contig, a.D, a.ds, a.status); break;
                case 2: unpack_unit<2>(s, st, &s.empty[stg], consumed, rows_contig, a.D, a.ds, a.status); break;
                case 3: unpack_unit<3>(s, st, &s.empty[stg], consumed, rows_contig, a.D, a.ds, a.status); break;
                default: unpack_unit<4>(s, st, &s.empty[stg], consumed, rows_contig, a.D, a.ds, a.status); break;
            }
        }
    }
    bulk_wait_all();
}
