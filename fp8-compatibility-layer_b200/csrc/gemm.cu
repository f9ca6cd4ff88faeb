// Tile GEMM on prepared fp16 activations (kernel b):
//
//   y[m,n] = xs[m] * smax[n] * sum_k x16[m,k] * (dec(codes[n,k]) * scale[n,k/G] / smax[n]) + bias[n]
//
// Computed transposed, D[n, m], so that the 128 rows of the tcgen05 MMA are WEIGHT rows: a CTA
// decodes each FP8 tile once and multiplies it against up to 256 activation rows, and small M
// (16..128) simply uses a narrower MMA instead of padding the 128-row dimension.
//
// Persistent CTAs (one per SM) walk the list of 128 x BN output tiles. K flows in 64-wide k-blocks
// through three shared-memory rings that never drain between tiles -- raw FP8 codes (deep: it
// hides HBM latency), activation tiles (their own ring with their own barriers, as deep as the
// tile width allows: an activation tile is requested when its slot is released and arrives an L2
// round trip later, so with only as many slots as decoded tiles that round trip, not the tensor
// core, paced narrow tiles), decoded fp16 weight tiles -- and the FP32 accumulators are
// double-buffered in tensor memory so the epilogue of a tile overlaps the main loop of the next.
// Warp roles:
//   warp 0       raw-code producer: one tiled TMA load per raw slot, 128 weight rows x 128
//                contiguous bytes (two k-blocks; 64 bytes when K is not a multiple of 128);
//   warp 2       activation producer: per k-block one load of the BN x 64 fp16 tile in the
//                128-byte swizzle; no multicast anywhere;
//   warp 1       tensor-memory allocation; one thread issues tcgen05.mma (kind::f16, M = 128,
//                N = BN, K = 16) four times per k-block and tcgen05.commit's the two tiles free;
//   warps 3..18  decode, in groups that take alternate k-blocks: 16 codes per thread per step to
//                fp16 (two codes per conversion instruction), the K-group scale folded in as
//                scale / rowmax (a packed fp16 multiply when the ratio is a power of two, else an
//                FP32 multiply with one fp16 rounding), written in the 128-byte-swizzled K-major
//                layout the MMA reads; fence.proxy.async, then mbarrier arrives;
//   warps 19..22 epilogue: tcgen05.ld the FP32 accumulators, apply smax[n], xs[m], bias[n], round
//                once to the output type and store (32 lanes = 32 consecutive n per m).
// No fp16 copy of the weights ever exists outside shared memory. Every mbarrier wait is bounded;
// a wait that runs out sets a status bit, and the thread keeps walking its loops without waiting
// so that every barrier is still met and the CTA ends.
#include <stdlib.h>

#include "common.cuh"

namespace tfp8b {

constexpr int GM_BM = 128;          // weight rows per tile = UMMA M = TMEM lanes
constexpr int GM_BK = 64;           // K per k-block: one 128-byte swizzle atom of fp16
constexpr int GM_DEC_WARPS = 16;
constexpr int GM_DEC_THREADS = GM_DEC_WARPS * 32;
// Decode groups (a kernel template parameter): group g decodes k-blocks g, g + NG, ...; a decode
// thread handles NG rows of its k-block. Two groups of eight warps everywhere, except four groups
// of four warps for tiles of at most 32 activation rows whose K-group scales sit in shared
// memory: there a k-block is a few hundred instructions of fixed cost per warp, and half as
// many warps per k-block pay it (eight decoded-tile slots, which only such narrow tiles leave room for).
constexpr int GM_DEC_WARP0 = 4;                        // warps 0..3: raw producer, MMA, activation producer, second MMA
constexpr int GM_EPI_WARP0 = GM_DEC_WARP0 + GM_DEC_WARPS;
constexpr int GM_THREADS = (GM_EPI_WARP0 + 4) * 32;
constexpr int GM_MAX_SLOTS = 8;     // per ring (decoded tiles, raw codes)
constexpr int GM_MAX_XSLOTS = 8;    // activation ring
constexpr int GM_MAX_DST = 8;       // output destinations of one launch (one per GPU of a tensor-parallel group)
constexpr int GM_HEADER = 2048;     // barriers, TMEM base, per-row scale reciprocals
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;    // decoded fp16 tile
constexpr int GM_RAW_BYTES = GM_BM * GM_BK;      // raw FP8 tile of one k-block
constexpr int GM_SMEM_MAX = 232448;              // 227 KB opt-in limit per CTA

struct GemmParams {
    int sc_row;               // bytes of one row's K-group scales kept in shared memory per tile, 0 = read from global
    const float* xs;
    const void* scale;
    const float* bias;
    void* y[GM_MAX_DST];      // output buffers: this GPU's and, for a fused gather, every peer's
    long long ldy, col0;      // row pitch of the outputs in elements; column where this call's N columns start
    int ndst;
    int push;                 // peers are served by the push warp (16-byte copies of whole tile rows), not by the epilogue
    int M, N, K, G, scale_kind, y_dt;
    int BN, tmem_cols, m_tiles, ntiles;
    int ns, sr, nx;      // slots of the decoded-tile ring, of the raw-code ring, of the activation ring
    int rb;              // k-blocks per raw slot: 2 (128 bytes per weight row and copy) or 1
    int x_bytes;         // one activation tile: BN x 64 fp16
    int ng;              // decode groups (the kernel's NG)
    int nmma;            // MMA-issuing threads; thread t takes k-blocks t, t + nmma, ... into its own accumulator
    int ks, nkbu;        // split-K: every tile is cut into ks units of nkbu k-blocks; ntiles counts units
    int span, span_total, nkbt;   // split-K by spans (span > 0): CTA b owns k-blocks [b * span, (b + 1) * span) of the
                         // tile-major sequence of all span_total k-blocks; a tile has nkbt of them
    float* ws;           // split-K: FP32 [M, N] workspace the units add their partial tiles into
};

struct GemmHeader {
    uint64_t full[GM_MAX_SLOTS], empty[GM_MAX_SLOTS];
    uint64_t raw_full[GM_MAX_SLOTS], raw_empty[GM_MAX_SLOTS];
    uint64_t x_full[GM_MAX_XSLOTS], x_empty[GM_MAX_XSLOTS];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sc_full[2], sc_empty[2];   // the tile's K-group scales in shared memory, double-buffered by unit parity
    uint32_t tmem_base;
    uint32_t tiles_stored;    // epilogue warps that have finished writing a tile to the local output (4 per tile)
    float binv[2][GM_BM];   // per weight row: 1 / max_g scale[n,g], double-buffered by tile parity
};
static_assert(sizeof(GemmHeader) <= GM_HEADER, "header too large");

// Build with -DTFP8B_GM_TRACE to record, for CTA 0, the SM clock at which each role passes each
// k-block (a diagnostic for pipeline tuning; the array is read with cudaMemcpyFromSymbol; rows 8
// and 9: when each raw slot's copy, and each k-block's MMAs, were seen complete by an idle warp). Row 0
// also holds, at indices 250 - 255: kernel entry, end of set-up, first epilogue's start and end,
// (unused), TMEM release.
#ifdef TFP8B_GM_TRACE
__device__ long long g_trace[10][256];
#define GM_TRACE(ev, idx) do { if (blockIdx.x == 0 && (idx) < 256) g_trace[ev][idx] = clock64(); } while (0)
#else
#define GM_TRACE(ev, idx) do { } while (0)
#endif

// ------------------------------------------------------------------ tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t r[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand in the 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart (stride byte offset), leading byte offset unused (1), descriptor
// version 1, layout type 2. The tile base must be 1024-byte aligned; stepping K by 16 fp16
// elements advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ uint4 gm_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void gm_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// max over one row's K-group scales, entries [g0, g1). The loads are independent and issued in
// batches (16-byte vectors where the row allows it): a one-load-at-a-time loop costs an L2 round
// trip per scale, which for 256 groups is longer than the tile's whole main loop.
__device__ __forceinline__ float row_scale_max(const void* scale, size_t row_off, int g0, int g1, int kind,
                                               uint32_t* bmax_out = nullptr) {
    const int esz = kind == TFP8B_SCALE_UE8M0 ? 1 : 4;
    const uint8_t* base = reinterpret_cast<const uint8_t*>(scale) + (row_off + g0) * esz;
    const int n = g1 - g0;
    const int per = 16 / esz;                                   // scales per 16-byte vector
    float mx = 0.f;
    uint32_t bmax = 0u;                                         // UE8M0: max of the exponent bytes (255 = NaN wins)
    int i = 0;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) {
        const uint4* v = reinterpret_cast<const uint4*>(base);
        const int nv = n / per;
        for (int j = 0; j < nv; j += 8) {
            uint4 t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = j + u < nv ? __ldg(v + j + u) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t w[4] = {t[u].x, t[u].y, t[u].z, t[u].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (kind == TFP8B_SCALE_UE8M0) {
                        const uint32_t m4 = __vmaxu4(w[e], __byte_perm(w[e], 0u, 0x4321));   // pairwise byte maxima
                        bmax = max(bmax, max(m4 & 0xFFu, (m4 >> 16) & 0xFFu));
                    } else {
                        mx = fmaxf(mx, __uint_as_float(w[e]));
                    }
                }
            }
        }
        i = nv * per;
    }
    for (; i < n; ++i) {
        if (kind == TFP8B_SCALE_UE8M0) bmax = max(bmax, static_cast<uint32_t>(base[i]));
        else mx = fmaxf(mx, reinterpret_cast<const float*>(base)[i]);
    }
    if (kind == TFP8B_SCALE_UE8M0) mx = n > 0 ? ue8m0_to_f32(bmax) : 0.f;
    if (bmax_out) *bmax_out = bmax;
    return mx;
}

// ------------------------------------------------------------------ the kernel
// OUT selects how a finished tile leaves the CTA; each form is a kernel of its own because the
// uncommon ones, merely present as untaken branches, slowed the plain one by 4 - 17 % (longer
// epilogue, different register allocation in the decode loop):
//   GM_OUT_PLAIN   one output [M, N], whole K                       (every ordinary linear layer)
//   GM_OUT_SPLITK  FP32 atomics into the workspace; units = (tile, K part)
//   GM_OUT_WINDOW  1..8 outputs with a row pitch and a column offset, element-wise stores
//   GM_OUT_PUSH    the same, peers served by the push warp from the local copy
constexpr int GM_OUT_PLAIN = 0, GM_OUT_SPLITK = 1, GM_OUT_WINDOW = 2, GM_OUT_PUSH = 3;

// SC: the tile's K-group scales are kept in shared memory (see the decode warps). A template
// parameter because the two ways of fetching scale ratios want different loop shapes: from global
// memory they are fetched four of the group's k-blocks ahead and the loop is unrolled by four;
// from shared memory one k-block ahead is enough, and the four-times smaller loop body matters:
// the roles of this kernel together are ~7000 instructions, far more than an instruction cache
// level close to the schedulers holds.
template <int FMT, int OUT, int SC, int NG>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
    static_assert(NG == 2 || NG == 4, "two or four decode groups");
    constexpr int GROUP_THREADS = GM_DEC_THREADS / NG, GROUP_WARPS = GM_DEC_WARPS / NG;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment of the tile buffers is required by the swizzled layouts.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    GemmHeader* hd = reinterpret_cast<GemmHeader*>(smem);
    if (threadIdx.x == 0) GM_TRACE(0, 250);
    uint8_t* stages = smem + GM_HEADER;                                   // decoded tiles, 16 KB each
    uint8_t* x_ring = stages + static_cast<size_t>(p.ns) * GM_A_BYTES;    // activation tiles
    uint8_t* raw_ring = x_ring + static_cast<size_t>(p.nx) * p.x_bytes;
    uint8_t* sc_cache = raw_ring + static_cast<size_t>(p.sr) * p.rb * GM_RAW_BYTES;   // [2][128 rows][sc_row bytes]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int raw_slot_bytes = p.rb * GM_RAW_BYTES;
    const int ng = p.K / p.G;
    // Unit i of this CTA is global unit blockIdx.x + i * gridDim.x = (tile, K part), the part the
    // fast index; within the tiles the activation-row tile is the fast index, so CTAs that run
    // together share one weight stripe through L2.
    // Split-K by spans: the k-blocks of all tiles form one tile-major sequence, and CTA b owns
    // [b * span, (b + 1) * span) of it, so every SM works equally long whatever the number of
    // tiles. The span is cut at tile boundaries into this CTA's units (at most three while
    // span >= a tile's k-blocks): the end of one tile, whole tiles, the start of another.
    constexpr bool SPLIT = OUT == GM_OUT_SPLITK;
    const bool spans = SPLIT && p.span > 0;
    const int sp_lo = spans ? static_cast<int>(blockIdx.x) * p.span : 0;
    const int sp_hi = spans ? min(sp_lo + p.span, p.span_total) : 0;
    const int sp_t0 = spans ? sp_lo / p.nkbt : 0;
    const int my_tiles = spans ? (sp_hi > sp_lo ? (sp_hi - 1) / p.nkbt - sp_t0 + 1 : 0)
                               : (p.ntiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    auto unit_of = [&](int i) { return static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x); };
    auto tile_of = [&](int i) { return spans ? sp_t0 + i : (SPLIT ? unit_of(i) / p.ks : unit_of(i)); };
    auto tile_m0 = [&](int i) { return (tile_of(i) % p.m_tiles) * p.BN; };
    auto tile_n0 = [&](int i) { return (tile_of(i) / p.m_tiles) * GM_BM; };
    // first k-block of the unit inside its tile, its number of k-blocks, and the k-blocks of the
    // CTA's earlier units
    auto unit_kb0 = [&](int i) { return spans ? max(sp_lo - (sp_t0 + i) * p.nkbt, 0) : (SPLIT ? (unit_of(i) % p.ks) * p.nkbu : 0); };
    auto unit_len = [&](int i) { return spans ? min(sp_hi, (sp_t0 + i + 1) * p.nkbt) - max(sp_lo, (sp_t0 + i) * p.nkbt) : p.nkbu; };
    auto unit_base = [&](int i) { return spans ? max((sp_t0 + i) * p.nkbt - sp_lo, 0) : i * p.nkbu; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.ns; ++s) {
            mbar_init(smem_u32(&hd->full[s]), GROUP_WARPS);          // the warps of the group that decoded it
            mbar_init(smem_u32(&hd->empty[s]), 1);
        }
        for (int s = 0; s < p.nx; ++s) {
            mbar_init(smem_u32(&hd->x_full[s]), 1);                     // the activation copy (bytes counted)
            mbar_init(smem_u32(&hd->x_empty[s]), 1);
        }
        for (int s = 0; s < p.sr; ++s) {
            mbar_init(smem_u32(&hd->raw_full[s]), 1);
            mbar_init(smem_u32(&hd->raw_empty[s]), GROUP_WARPS * p.rb);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&hd->acc_full[b]), p.nmma);
            mbar_init(smem_u32(&hd->acc_empty[b]), 4);
            mbar_init(smem_u32(&hd->sc_full[b]), 1);                    // the scale copy (bytes counted)
            mbar_init(smem_u32(&hd->sc_empty[b]), GM_DEC_WARPS);
        }
        hd->tiles_stored = 0u;
        mbar_fence_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&hd->tmem_base), static_cast<uint32_t>(p.tmem_cols));
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) GM_TRACE(0, 251);
    const uint32_t tmem_base = hd->tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------------- raw-code producer
        if (lane == 0) {
            // One activation tile only: the weight stripe is read once, keep it out of L2's way.
            // Several tiles: the CTAs of the other tiles read the same stripe from L2 next.
            const uint64_t pol_w = p.m_tiles == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
            int slot = 0;
            uint32_t phase = 1;               // ring position (no divisions): the first pass over the ring does not wait
            bool ok = true, first_pass = true;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int n0 = tile_n0(i), kb0 = unit_kb0(i), nkb = unit_len(i);
                if (SC) {
                    // The K-group scales of the unit's weight rows, one bulk copy into the buffer of
                    // the unit's parity, issued before the unit's codes: a dozen k-blocks ahead of
                    // the decode warps, which then never wait for a scale. (Fetched by the decode
                    // warps themselves at the start of a tile, the loads -- demand misses queued
                    // behind the megabytes of codes this kernel keeps in flight -- cost 5 us per tile.)
                    const int b = i & 1;
                    if (i >= 2 && !mbar_wait(smem_u32(&hd->sc_empty[b]), static_cast<uint32_t>(((i >> 1) - 1) & 1), STATUS_GEMM_WAIT)) { ok = false; break; }
                    const uint32_t bytes = static_cast<uint32_t>(min(GM_BM, p.N - n0) * p.sc_row);
                    const uint32_t bar = smem_u32(&hd->sc_full[b]);
                    mbar_expect_tx(bar, bytes);
                    bulk_g2s(smem_u32(sc_cache + static_cast<size_t>(b) * GM_BM * p.sc_row),
                             reinterpret_cast<const uint8_t*>(p.scale) + static_cast<size_t>(n0) * p.sc_row, bytes, bar, l2_policy_evict_normal());
                }
                for (int kb = 0; kb < nkb; kb += p.rb) {
                    if (!first_pass && !mbar_wait(smem_u32(&hd->raw_empty[slot]), phase, STATUS_GEMM_WAIT)) { ok = false; break; }
                    GM_TRACE(0, unit_base(i) + kb);
                    const uint32_t bar = smem_u32(&hd->raw_full[slot]);
                    const uint32_t dst = smem_u32(raw_ring + static_cast<size_t>(slot) * raw_slot_bytes);
                    mbar_expect_tx(bar, static_cast<uint32_t>(raw_slot_bytes));
                    if (p.rb == 2) tma_load_3d(dst, &tm_w, 0, n0, (kb0 + kb) >> 1, bar, pol_w);     // [row][128 bytes]
                    else tma_load_2d(dst, &tm_w, (kb0 + kb) * GM_BK, n0, bar, pol_w);               // [row][64 bytes]
                    if (++slot == p.sr) { slot = 0; phase ^= 1u; first_pass = false; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ---------------------------------------------------------------- activation producer
        if (lane == 0) {
            const uint64_t pol_x = l2_policy_evict_last();
            int slot = 0;
            uint32_t phase = 1;
            bool ok = true, first_pass = true;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int m0 = tile_m0(i), kb0 = unit_kb0(i), nkb = unit_len(i);
                for (int kb = 0; kb < nkb; ++kb) {
                    if (!first_pass && !mbar_wait(smem_u32(&hd->x_empty[slot]), phase, STATUS_GEMM_WAIT)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&hd->x_full[slot]);
                    mbar_expect_tx(bar, static_cast<uint32_t>(p.x_bytes));
                    tma_load_2d(smem_u32(x_ring + static_cast<size_t>(slot) * p.x_bytes), &tm_x, (kb0 + kb) * GM_BK, m0, bar, pol_x);
                    if (++slot == p.nx) { slot = 0; phase ^= 1u; first_pass = false; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || (warp == 3 && p.nmma == 2)) {
        // ---------------------------------------------------------------- MMA issuer(s)
        // tcgen05.mma issue is paced by the tensor pipe, and everything else the issuing thread does
        // per k-block (the barrier wait, the fence, the commit, its bookkeeping) is a gap in which
        // the pipe can run dry. Two measures: the barrier of the thread's NEXT k-block is polled in
        // the middle of the current k-block's four MMAs, while two of them are still queued; and
        // for narrow tiles, where an MMA is short, two threads take alternate k-blocks of the
        // CTA's stream, each into an accumulator of its own (the epilogue adds the two). At
        // BN = 256 one double-buffered accumulator fills tensor memory and one thread issues.
        if (lane == 0) {
            // D fp32, A/B fp16, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(p.BN >> 3) << 17) | (static_cast<uint32_t>(GM_BM >> 4) << 24);
            const int t = warp == 1 ? 0 : 1;
            // this thread's cursors in the decoded-tile ring and in the activation ring: byte
            // offset of the slot, offset of its barriers, parity to wait for
            const uint32_t a_step = static_cast<uint32_t>(p.nmma * GM_A_BYTES), a_ring = static_cast<uint32_t>(p.ns * GM_A_BYTES);
            const uint32_t x_step = static_cast<uint32_t>(p.nmma * p.x_bytes), x_ringb = static_cast<uint32_t>(p.nx * p.x_bytes);
            const uint32_t stages_u32 = smem_u32(stages), xring_u32 = smem_u32(x_ring);
            uint32_t a_off = static_cast<uint32_t>(t * GM_A_BYTES), a_bar = static_cast<uint32_t>(t * 8), a_par = 0;
            uint32_t x_off = static_cast<uint32_t>(t * p.x_bytes), x_bar = static_cast<uint32_t>(t * 8), x_par = 0;
            const uint32_t full0 = smem_u32(&hd->full[0]), empty0 = smem_u32(&hd->empty[0]);
            const uint32_t xfull0 = smem_u32(&hd->x_full[0]), xempty0 = smem_u32(&hd->x_empty[0]);
            int next = t;                     // CTA-wide number of this thread's next k-block
            bool ok = true, ready = false;    // ready: the next k-block's barriers were already seen complete
            uint64_t da = umma_desc_sw128(stages_u32 + a_off), db = umma_desc_sw128(xring_u32 + x_off);
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int buf = i & 1;
                // the accumulator buffer must have been drained by the epilogue of tile i - 2
                if (i >= 2) ok = mbar_wait(smem_u32(&hd->acc_empty[buf]), ((i >> 1) - 1) & 1, STATUS_GEMM_WAIT);
                if (!ok) break;
                const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>((buf * p.nmma + t) * p.BN);
                uint32_t accumulate = 0u;
                const int nkb = unit_len(i), base = unit_base(i);
                int kb = next - base;
                for (; kb < nkb; kb += p.nmma) {
                    GM_TRACE(5, base + kb);
                    if (!ready) ok = mbar_wait(full0 + a_bar, a_par, STATUS_GEMM_WAIT) && mbar_wait(xfull0 + x_bar, x_par, STATUS_GEMM_WAIT);
                    if (!ok) break;
                    GM_TRACE(3, base + kb);
                    tc_fence_after();
                    tc_mma_f16(tmem_acc, da, db, idesc, accumulate);
                    tc_mma_f16(tmem_acc, da + 2, db + 2, idesc, 1u);
                    // while those two are queued: move on to this thread's next k-block, look at its
                    // barriers once and build its descriptors
                    const uint32_t cur_empty = empty0 + a_bar, cur_xempty = xempty0 + x_bar;
                    const uint64_t da_cur = da, db_cur = db;
                    a_off += a_step; a_bar += static_cast<uint32_t>(p.nmma * 8);
                    if (a_off >= a_ring) { a_off -= a_ring; a_bar -= static_cast<uint32_t>(p.ns * 8); a_par ^= 1u; }
                    x_off += x_step; x_bar += static_cast<uint32_t>(p.nmma * 8);
                    if (x_off >= x_ringb) { x_off -= x_ringb; x_bar -= static_cast<uint32_t>(p.nx * 8); x_par ^= 1u; }
                    ready = mbar_try_wait(full0 + a_bar, a_par) && mbar_try_wait(xfull0 + x_bar, x_par);
                    da = umma_desc_sw128(stages_u32 + a_off); db = umma_desc_sw128(xring_u32 + x_off);
                    tc_mma_f16(tmem_acc, da_cur + 4, db_cur + 4, idesc, 1u);
                    tc_mma_f16(tmem_acc, da_cur + 6, db_cur + 6, idesc, 1u);
                    GM_TRACE(6, base + kb);
                    tc_commit(cur_empty);             // both slots are free once these MMAs have read them
                    tc_commit(cur_xempty);
                    GM_TRACE(4, base + kb);
                    accumulate = 1u;
                }
                next = base + kb;
                if (ok) tc_commit(smem_u32(&hd->acc_full[buf]));
            }
        }
        __syncwarp();
    } else if (warp >= GM_DEC_WARP0 && warp < GM_EPI_WARP0) {
        // ---------------------------------------------------------------- decode warps
        // The CTA's k-blocks are numbered through all its tiles; group g owns numbers g, g + NG, ...
        // so NG k-blocks are in decode at once and a group's fixed costs per k-block (barrier
        // round trips, the proxy fence) overlap another group's work. The loop is kept lean on
        // purpose (32-bit shared addresses, per-thread offsets computed once, ring cursors
        // advanced by addition): with K-group scales this role is bound by instruction issue.
        constexpr int RPT = NG;                      // rows per decode thread and k-block (128 rows x 4 chunks)
        constexpr int RSTEP = GM_BM / RPT;           // distance between a thread's rows
        const int td = threadIdx.x - GM_DEC_WARP0 * 32;   // 0 .. GM_DEC_THREADS-1
        const int group = td / GROUP_THREADS;
        const int tg = td % GROUP_THREADS;
        const int c = tg & 3;                        // 16-code chunk of the 64-wide K block
        // Rows r0 + RSTEP * h. The 8 threads of a quarter-warp (one shared-memory wavefront of
        // a 16-byte access) work on rows R and R ^ 5 of the warp's 8: the two rows differ in bit
        // 0 and in bit 2 of the index, so that both the reads of the swizzled raw slot (chunks
        // (4 half + c) ^ row: the halves differ through bit 2) and the stores into the swizzled
        // decoded tile (chunks 2c ^ row: odd and even through bit 0) touch 8 different chunks.
        const int rr = (tg >> 2) & 7;
        const int r0 = (tg >> 5) * 8 + ((rr & 1) ? ((rr >> 1) ^ 5) : (rr >> 1));
        uint32_t roff[RPT], aoff0[RPT], aoff1[RPT];  // this thread's byte offsets inside a raw slot / a decoded tile
#pragma unroll
        for (int h2 = 0; h2 < RPT; ++h2) {
            const uint32_t r = static_cast<uint32_t>(r0 + RSTEP * h2);
            roff[h2] = p.rb == 2 ? r * 128u + ((static_cast<uint32_t>(c) ^ (r & 7u)) << 4) : r * 64u + static_cast<uint32_t>(c) * 16u;
            aoff0[h2] = r * 128u + (((2u * c) ^ (r & 7u)) << 4);
            aoff1[h2] = r * 128u + (((2u * c + 1u) ^ (r & 7u)) << 4);
        }
        const uint32_t stages_u32 = smem_u32(stages), raw_u32 = smem_u32(raw_ring);
        const uint32_t full0 = smem_u32(&hd->full[0]), empty0 = smem_u32(&hd->empty[0]);
        const uint32_t rfull0 = smem_u32(&hd->raw_full[0]), rempty0 = smem_u32(&hd->raw_empty[0]);
        // ring cursors of the group's next k-block: byte offset of its stage / raw slot, the offset
        // of their barriers, the parity to wait for
        const uint32_t a_step = static_cast<uint32_t>(NG * GM_A_BYTES), a_ring = static_cast<uint32_t>(p.ns * GM_A_BYTES);
        const uint32_t r_slots = static_cast<uint32_t>(NG / p.rb);           // raw slots between the group's k-blocks
        const uint32_t r_step = r_slots * raw_slot_bytes, r_ring = static_cast<uint32_t>(p.sr) * raw_slot_bytes;
        uint32_t a_off = static_cast<uint32_t>(group * GM_A_BYTES), a_bar = static_cast<uint32_t>(group * 8), a_par = 0;
        uint32_t r_off = static_cast<uint32_t>(group / p.rb) * raw_slot_bytes, r_bar = static_cast<uint32_t>(group / p.rb) * 8u, r_par = 0;
        int done = group;                            // CTA-wide number of the group's next k-block
        bool ok = true;
        const bool e8 = p.scale_kind == TFP8B_SCALE_UE8M0;
        // K-group of a k-block: (kb * 2 + c / 2) 32-code units / (G / 32); a shift when that is a power of two
        const int g32 = p.G / 32;
        const int g_shift = (g32 & (g32 - 1)) == 0 ? __ffs(g32) - 1 : -1;
        constexpr int PF = SC ? 1 : 4;               // the group's k-blocks whose scale ratios are fetched ahead
        for (int i = 0; i < my_tiles; ++i) {
            const int n0 = tile_n0(i);
            // per row: 1 / max_g scale (float scales) or the largest exponent byte (UE8M0)
            float binv[RPT];
            int bmax[RPT];
            size_t srow[RPT];
#pragma unroll
            for (int h2 = 0; h2 < RPT; ++h2) {
                binv[h2] = 1.f;
                bmax[h2] = 0;
                srow[h2] = static_cast<size_t>(min(n0 + r0 + RSTEP * h2, p.N - 1)) * ng;
            }
            // K-group scales of the tile. A scale read from global memory in the k-loop is a demand
            // miss that queues behind the megabytes of weight tiles this very kernel keeps in flight:
            // measured, it comes back about 2.4 us later, and with the ratios fetched eight k-blocks
            // ahead that latency -- not HBM bandwidth, not the tensor core -- set the pace of narrow
            // tiles (0.3 us per k-block whatever the width). So where a row's scales are short
            // enough, the producer copies the unit's scales into shared memory ahead of its codes
            // (double-buffered by unit parity: a group may already be in the next unit while the
            // other finishes this one), and the k-loop reads them from there. Rows past N (the last
            // tile) read the last row's scales.
            const uint8_t* sc = sc_cache + static_cast<size_t>(i & 1) * GM_BM * p.sc_row;
            uint32_t sc_off[RPT];                                                   // this thread's rows in it
#pragma unroll
            for (int h2 = 0; h2 < RPT; ++h2) sc_off[h2] = static_cast<uint32_t>(min(r0 + RSTEP * h2, p.N - 1 - n0) * p.sc_row);
            // UE8M0 scales cached for the tile: whether EVERY ratio of the warp's rows is a normal
            // fp16 power of two (exponent bytes within 14 of the row maximum) is known once per
            // tile, and the k-loop needs neither the range test nor a vote per k-block.
            bool tile_fast = true;
            if (ng > 1 && SC) {
                const int vpr = p.sc_row >> 4;                                      // 16-byte vectors per row
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->sc_full[i & 1]), static_cast<uint32_t>((i >> 1) & 1), STATUS_GEMM_WAIT));
                if (tg == 0) GM_TRACE(1, 200 + 2 * i);
                // Row maximum (and, UE8M0, minimum) of the scales: the four threads that share a
                // row (c = 0..3, neighbouring lanes) take every fourth 16-byte piece and combine by
                // shuffles; bytes are reduced four at a time.
#pragma unroll
                for (int h2 = 0; h2 < RPT; ++h2) {
                    const uint8_t* rowp = sc + sc_off[h2];
                    float mx = 0.f;
                    uint32_t m4 = 0u, n4 = 0xFFFFFFFFu;
                    for (int j = c; j < vpr; j += 4) {
                        const uint4 t = *reinterpret_cast<const uint4*>(rowp + j * 16);
                        if (e8) {
                            m4 = __vmaxu4(m4, __vmaxu4(__vmaxu4(t.x, t.y), __vmaxu4(t.z, t.w)));
                            n4 = __vminu4(n4, __vminu4(__vminu4(t.x, t.y), __vminu4(t.z, t.w)));
                        } else {
                            mx = fmaxf(mx, fmaxf(fmaxf(__uint_as_float(t.x), __uint_as_float(t.y)), fmaxf(__uint_as_float(t.z), __uint_as_float(t.w))));
                        }
                    }
#pragma unroll
                    for (int o = 1; o < 4; o <<= 1) {
                        if (e8) {
                            m4 = __vmaxu4(m4, __shfl_xor_sync(0xffffffffu, m4, o));
                            n4 = __vminu4(n4, __shfl_xor_sync(0xffffffffu, n4, o));
                        } else {
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                        }
                    }
                    m4 = __vmaxu4(m4, m4 >> 16); m4 = __vmaxu4(m4, m4 >> 8);
                    n4 = __vminu4(n4, n4 >> 16); n4 = __vminu4(n4, (n4 >> 8) | 0xFF000000u);
                    const uint32_t bm = m4 & 0xFFu, bn = n4 & 0xFFu;
                    binv[h2] = e8 ? __uint_as_float(bm) : (mx > 0.f ? 1.f / mx : 0.f);
                    bmax[h2] = static_cast<int>(bm);
                    // smallest exponent byte of the row against the largest: decides the fold form for the tile
                    if (e8) tile_fast = tile_fast && static_cast<int>(bm) - static_cast<int>(bn) <= 14;
                }
                if (tg == 0) GM_TRACE(1, 201 + 2 * i);
                tile_fast = e8 && __all_sync(0xffffffffu, tile_fast);
            } else if (ng > 1) {
                // row maxima of the K-group scales: GM_DEC_THREADS / 128 threads share a row
                constexpr int TPR = GM_DEC_THREADS / GM_BM;
                const int row = td / TPR, part = td % TPR;
                const size_t off = static_cast<size_t>(min(n0 + row, p.N - 1)) * ng;
                const int g0 = (ng * part) / TPR, g1 = (ng * (part + 1)) / TPR;
                uint32_t bm = 0u;
                float mx = row_scale_max(p.scale, off, g0, g1, p.scale_kind, &bm);
#pragma unroll
                for (int o = 1; o < TPR; o <<= 1) {
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    bm = max(bm, __shfl_xor_sync(0xffffffffu, bm, o));
                }
                if (part == 0) hd->binv[i & 1][row] = e8 ? __uint_as_float(bm) : (mx > 0.f ? 1.f / mx : 0.f);
                named_barrier_sync(1, GM_DEC_THREADS);
#pragma unroll
                for (int h2 = 0; h2 < RPT; ++h2) {
                    binv[h2] = hd->binv[i & 1][r0 + RSTEP * h2];
                    bmax[h2] = static_cast<int>(__float_as_uint(binv[h2]));
                }
            }
            // this group's k-blocks inside the tile: first, first + NG, ... (nloc of them)
            const int nkb = unit_len(i), ubase = unit_base(i);
            const int first = done - ubase;
            const int nloc = first < nkb ? (nkb - first + NG - 1) / NG : 0;
            const int kabs = unit_kb0(i) + first;                                  // absolute k-block of the group's first one
            const uint32_t half_off = (p.rb == 2 && (kabs & 1)) ? 64u : 0u;        // NG is even: the parity of kb is fixed
            // The fold factor scale / rowmax of this thread's rows for PF of the group's k-blocks,
            // loaded one batch ahead of their use (a global load inside the k-block loop would stall
            // every decode warp for an L2 round trip). UE8M0: the factor is 2^e with e the byte
            // difference, kept as an integer; float scales: the factor itself, as float bits.
            auto load_ratios = [&](int l0, uint32_t (*dst)[RPT]) {
#pragma unroll
                for (int j = 0; j < PF; ++j) {
#pragma unroll
                    for (int h2 = 0; h2 < RPT; ++h2) dst[j][h2] = e8 ? 0u : 0x3F800000u;
                    if (ng > 1 && l0 + j < nloc) {
                        const int u32 = (kabs + (l0 + j) * NG) * 2 + (c >> 1);
                        const int gi = min(g_shift >= 0 ? (u32 >> g_shift) : (u32 / g32), ng - 1);
                        if (SC) {
#pragma unroll
                            for (int h2 = 0; h2 < RPT; ++h2) {
                                const uint8_t* rowp = sc + sc_off[h2];
                                if (e8) dst[j][h2] = static_cast<uint32_t>(static_cast<int>(rowp[gi]) - bmax[h2]);
                                else dst[j][h2] = __float_as_uint(reinterpret_cast<const float*>(rowp)[gi] * binv[h2]);
                            }
                        } else {
#pragma unroll
                            for (int h2 = 0; h2 < RPT; ++h2) {
                                if (e8) dst[j][h2] = static_cast<uint32_t>(static_cast<int>(reinterpret_cast<const uint8_t*>(p.scale)[srow[h2] + gi]) - bmax[h2]);
                                else dst[j][h2] = __float_as_uint(reinterpret_cast<const float*>(p.scale)[srow[h2] + gi] * binv[h2]);
                            }
                        }
                    }
                }
            };
            uint32_t rcur[PF][RPT], rnext[PF][RPT];
            load_ratios(0, rcur);
            for (int l0 = 0; l0 < nloc; l0 += PF) {
                load_ratios(l0 + PF, rnext);
#pragma unroll
                for (int j = 0; j < PF; ++j) {
                    if (l0 + j >= nloc) break;
                    const uint32_t st = stages_u32 + a_off, raw = raw_u32 + r_off;
                    const uint32_t bar_full = full0 + a_bar, bar_empty = empty0 + a_bar;
                    const uint32_t bar_rfull = rfull0 + r_bar, bar_rempty = rempty0 + r_bar;
                    const uint32_t apar = a_par, rpar = r_par;
                    const bool fresh = done < p.ns;          // the stage's first use: nothing to wait for
                    done += NG;
                    a_off += a_step; a_bar += NG * 8;
                    if (a_off >= a_ring) { a_off -= a_ring; a_bar -= static_cast<uint32_t>(p.ns * 8); a_par ^= 1u; }
                    r_off += r_step; r_bar += r_slots * 8u;
                    if (r_off >= r_ring) { r_off -= r_ring; r_bar -= static_cast<uint32_t>(p.sr * 8); r_par ^= 1u; }
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_rfull, rpar, STATUS_GEMM_WAIT));
                    if (ok && !fresh) ok = __all_sync(0xffffffffu, mbar_wait(bar_empty, apar ^ 1u, STATUS_GEMM_WAIT));
                    if (!ok) continue;
                    if (tg == 0) GM_TRACE(1, ubase + first + (l0 + j) * NG);
                    // all loads, then all conversions, then all stores: the rows of a thread are
                    // independent, and kept apart like this their latencies overlap
                    uint32_t h[RPT][8];
                    {
                        uint4 q[RPT];
#pragma unroll
                        for (int h2 = 0; h2 < RPT; ++h2) q[h2] = gm_lds128(raw + (roff[h2] ^ half_off));   // the k-block's half: chunk bit 2
#pragma unroll
                        for (int h2 = 0; h2 < RPT; ++h2) {
                            const uint32_t w[4] = {q[h2].x, q[h2].y, q[h2].z, q[h2].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) dec4_split<FMT>(w[e], h[h2][2 * e], h[h2][2 * e + 1]);
                        }
                    }
                    if (ng > 1) {
                        // Fold scale / rowmax in. A power of two inside fp16's normal range (1 included)
                        // is one packed multiply with the same rounding as the general path (an FP32
                        // multiply and one fp16 rounding); the choice is made for the whole warp.
                        // UE8M0 factors are powers of two by construction: 2^e, e <= 0, whose fp16
                        // bit pattern is (e + 15) << 10 while e >= -14.
                        bool fast;
                        if (SC && e8) {
                            fast = tile_fast;
                        } else {
                            bool pow2 = true;
#pragma unroll
                            for (int h2 = 0; h2 < RPT; ++h2) {
                                const uint32_t rb = rcur[j][h2];
                                pow2 = pow2 && (e8 ? static_cast<int>(rb) >= -14
                                                   : ((rb & 0x007FFFFFu) == 0u && rb >= 0x38800000u && rb <= 0x47000000u));
                            }
                            fast = __all_sync(0xffffffffu, pow2);
                        }
                        if (fast) {
#pragma unroll
                            for (int h2 = 0; h2 < RPT; ++h2) {
                                const uint32_t rb = rcur[j][h2];
                                // fp16 bits of the factor, in both halves: from the exponent directly
                                const uint32_t hb = e8 ? (rb + 15u) << 10 : ((rb >> 23) - 112u) << 10;
                                const uint32_t r2u = hb * 0x00010001u;
                                const __half2 r2 = *reinterpret_cast<const __half2*>(&r2u);
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    __half2 o = __hmul2(*reinterpret_cast<__half2*>(&h[h2][e]), r2);
                                    h[h2][e] = *reinterpret_cast<uint32_t*>(&o);
                                }
                            }
                        } else {
#pragma unroll
                            for (int h2 = 0; h2 < RPT; ++h2) {
                                const uint32_t rb = rcur[j][h2];
                                const float rt = e8 ? __uint_as_float(static_cast<uint32_t>(max(static_cast<int>(rb) + 127, 0)) << 23)
                                                    : __uint_as_float(rb);
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h[h2][e]));
                                    __half2 o = __floats2half2_rn(f.x * rt, f.y * rt);
                                    h[h2][e] = *reinterpret_cast<uint32_t*>(&o);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int h2 = 0; h2 < RPT; ++h2) {
                        gm_sts128(st + aoff0[h2], h[h2][0], h[h2][1], h[h2][2], h[h2][3]);
                        gm_sts128(st + aoff1[h2], h[h2][4], h[h2][5], h[h2][6], h[h2][7]);
                    }
                    if (tg == 0) GM_TRACE(7, ubase + first + (l0 + j) * NG);
                    fence_proxy_async_smem();        // generic-proxy stores -> visible to the tensor core
                    __syncwarp();
                    if (tg == 0) GM_TRACE(2, ubase + first + (l0 + j) * NG);
                    if (lane == 0) {
                        mbar_arrive(bar_full);
                        mbar_arrive(bar_rempty);     // this warp has read its part of the raw slot
                    }
                }
#pragma unroll
                for (int j = 0; j < PF; ++j)
#pragma unroll
                    for (int h2 = 0; h2 < RPT; ++h2) rcur[j][h2] = rnext[j][h2];
            }
            if (SC) {                                    // this warp has read the unit's scales for the last time
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&hd->sc_empty[i & 1]));
            }
        }
    } else if (OUT == GM_OUT_PUSH && warp == 3) {
        // ---------------------------------------------------------------- push warp (fused gather)
        // The accumulator is transposed (a warp owns 32 output columns), so an epilogue store is
        // 64 contiguous bytes: too small to keep NVLink busy, and the epilogue would stall the
        // MMA behind it. The epilogue therefore writes the tile to the LOCAL output only, and this
        // warp copies each finished tile to the peers from there (L2-hot), 16 bytes per lane,
        // whole 256-byte tile rows per request, while the next tile's main loop runs. (Warp 3 is
        // the second MMA issuer of narrow tiles; they keep the element-wise peer stores.)
        {
            const int esz = p.y_dt == TFP8B_F32 ? 4 : 2;
            const long long t0 = clock64();
            bool ok = true;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const uint32_t need = 4u * static_cast<uint32_t>(i + 1);
                while (*reinterpret_cast<volatile uint32_t*>(&hd->tiles_stored) < need) {      // bounded wait
                    __nanosleep(200);
                    if (clock64() - t0 > (1ll << 34)) { ok = false; break; }
                }
                if (!ok) { if (lane == 0) atomicOr(&g_status, STATUS_GEMM_WAIT); break; }
                __threadfence_block();
                const int m0 = tile_m0(i), n0 = tile_n0(i);
                const int rows = min(p.BN, p.M - m0), cols = min(GM_BM, p.N - n0);
                const int cpr = cols * esz / 16;                                    // 16-byte chunks per tile row
                const int total = rows * cpr;
                const size_t row_pitch = static_cast<size_t>(p.ldy) * esz;
                const size_t base = (static_cast<size_t>(m0) * p.ldy + p.col0 + n0) * esz;
                const uint8_t* src = reinterpret_cast<const uint8_t*>(p.y[0]) + base;
                for (int c0 = lane; c0 < total; c0 += 32 * 4) {
                    uint4 v[4];
                    size_t off[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = c0 + 32 * u;
                        const int r = c / cpr, k = c - r * cpr;
                        off[u] = static_cast<size_t>(r) * row_pitch + static_cast<size_t>(k) * 16;
                        if (c < total) v[u] = __ldcg(reinterpret_cast<const uint4*>(src + off[u]));
                    }
                    for (int d = 1; d < p.ndst; ++d) {
                        uint8_t* dst = reinterpret_cast<uint8_t*>(p.y[d]) + base;
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            if (c0 + 32 * u < total) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
                    }
                }
            }
        }
    } else if (warp >= GM_EPI_WARP0) {
        // ---------------------------------------------------------------- epilogue warps
        const int quarter = warp & 3;                           // TMEM lanes this warp may read
        const int row = quarter * 32 + lane;
        void* const y0 = p.y[0];
        // 16-bit outputs whose rows are whole 16-byte chunks: the lanes transpose among themselves
        // and store 8 columns at a time (else one element per store)
        const bool wide16 = OUT == GM_OUT_PLAIN && p.y_dt != TFP8B_F32 && (p.N & 7) == 0 && (reinterpret_cast<uintptr_t>(y0) & 15u) == 0;
        const bool b0 = lane & 1, b1 = lane & 2, b2 = lane & 4;
        bool ok = true;
#ifdef TFP8B_GM_TRACE
        // Two of these warps, idle until the first unit's accumulator is complete, watch that
        // unit's barriers: row 8 = when each raw slot's copy landed, row 9 = when the MMAs of each
        // k-block had finished (its decoded tile was free again).
        if (blockIdx.x == 0 && my_tiles > 0) {
            const int total = unit_len(0);
            if (warp == GM_EPI_WARP0) {
                int slot = 0;
                uint32_t phase = 0;
                for (int n = 0; n < total && n < 256; n += p.rb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->raw_full[slot]), phase, STATUS_GEMM_WAIT))) break;
                    if (lane == 0) g_trace[8][n] = clock64();
                    if (++slot == p.sr) { slot = 0; phase ^= 1u; }
                }
            } else if (warp == GM_EPI_WARP0 + 1) {
                for (int n = 0; n < total && n < 256; ++n) {
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->empty[n % p.ns]), static_cast<uint32_t>((n / p.ns) & 1), STATUS_GEMM_WAIT))) break;
                    if (lane == 0) g_trace[9][n] = clock64();
                }
            }
        }
#endif
        for (int i = 0; i < my_tiles; ++i) {
            const int buf = i & 1;
            const int m0 = tile_m0(i), n0 = tile_n0(i);
            const int n = n0 + row;
            const bool live = n < p.N;
            const size_t off = static_cast<size_t>(min(n, p.N - 1)) * ng;
            const float sm = ng == 1 ? load_scale(p.scale, off, p.scale_kind) : row_scale_max(p.scale, off, 0, ng, p.scale_kind);
            const float b = (p.bias && live) ? __ldg(p.bias + n) : 0.f;
            // Activation-row scales of the whole tile, fetched before the accumulator is waited
            // for: register k of lane l holds the scale of row m0 + 32 k + l (coalesced read-only
            // loads), handed out by shuffles. Every CTA of a wave asks for the same few lines at
            // the same moment, so a load costs well over a thousand cycles here; fetched where
            // they are used (and as ordinary loads, which may not pass the stores through the
            // untyped output pointer) they made up most of the epilogue's time.
            float xv[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int m = m0 + 32 * k + lane;
                xv[k] = (OUT != GM_OUT_SPLITK && 32 * k < p.BN && m < p.M) ? __ldg(p.xs + m) : 0.f;
            }
            float xcur = 0.f;
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->acc_full[buf]), (i >> 1) & 1, STATUS_GEMM_WAIT));
            if (!ok) continue;
            tc_fence_after();
            if (threadIdx.x == GM_EPI_WARP0 * 32) GM_TRACE(0, 252);
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * p.nmma * p.BN);
            for (int col = 0; col < p.BN; col += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + col, v);
                if ((col & 16) == 0) {                           // register col / 32, selected without indexing
                    const int k = col >> 5;
                    const float a0 = (k & 1) ? xv[1] : xv[0], a1 = (k & 1) ? xv[3] : xv[2];
                    const float a2 = (k & 1) ? xv[5] : xv[4], a3 = (k & 1) ? xv[7] : xv[6];
                    const float b0 = (k & 2) ? a1 : a0, b1 = (k & 2) ? a3 : a2;
                    xcur = (k & 4) ? b1 : b0;
                }
                tmem_ld_wait();
                for (int a = 1; a < p.nmma; ++a) {               // the second issuer's accumulator
                    uint32_t u[16];
                    tmem_ld16(taddr + a * p.BN + col, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                }
                const int mrows = min(16, p.M - (m0 + col));     // may be <= 0 in the last activation tile
                float val[16];
                if (OUT == GM_OUT_SPLITK) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) val[j] = __uint_as_float(v[j]) * sm;
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        val[j] = fmaf(__uint_as_float(v[j]) * sm, __shfl_sync(0xffffffffu, xcur, (col & 16) + j), b);
                }
                if (OUT == GM_OUT_PLAIN) {
                    const size_t at0 = static_cast<size_t>(m0 + col) * p.N + n;
                    if (wide16) {
                        // Three exchange steps (lane distance 1, 2, 4) turn "16 rows of one
                        // column per lane" into "2 rows of 8 consecutive columns per lane":
                        // two 16-byte stores instead of sixteen 2-byte ones.
                        uint32_t w1[8];                       // row 2t + b0: columns 2 (lane / 2) + {0, 1}
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const float got = __shfl_xor_sync(0xffffffffu, b0 ? val[2 * t] : val[2 * t + 1], 1);
                            const float lo = b0 ? got : val[2 * t], hi = b0 ? val[2 * t + 1] : got;
                            if (p.y_dt == TFP8B_F16) { __half2 h = __floats2half2_rn(lo, hi); w1[t] = *reinterpret_cast<uint32_t*>(&h); }
                            else { __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); w1[t] = *reinterpret_cast<uint32_t*>(&h); }
                        }
                        uint32_t w2[4][2];                    // row 4u + 2 b1 + b0: columns 4 (lane / 4) + {0..3}
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t got = __shfl_xor_sync(0xffffffffu, b1 ? w1[2 * u] : w1[2 * u + 1], 2);
                            const uint32_t mine = b1 ? w1[2 * u + 1] : w1[2 * u];
                            w2[u][0] = b1 ? got : mine;
                            w2[u][1] = b1 ? mine : got;
                        }
                        const int gcol = n0 + quarter * 32 + 8 * (lane >> 3);        // first of this lane's 8 columns
                        uint16_t* yb = reinterpret_cast<uint16_t*>(y0) + static_cast<size_t>(m0 + col + (lane & 7)) * p.N + gcol;
#pragma unroll
                        for (int q = 0; q < 2; ++q) {         // row 8q + (lane & 7): columns 8 (lane / 8) + {0..7}
                            const uint32_t g0 = __shfl_xor_sync(0xffffffffu, b2 ? w2[2 * q][0] : w2[2 * q + 1][0], 4);
                            const uint32_t g1 = __shfl_xor_sync(0xffffffffu, b2 ? w2[2 * q][1] : w2[2 * q + 1][1], 4);
                            const uint32_t k0 = b2 ? w2[2 * q + 1][0] : w2[2 * q][0], k1 = b2 ? w2[2 * q + 1][1] : w2[2 * q][1];
                            const uint4 out = b2 ? make_uint4(g0, g1, k0, k1) : make_uint4(k0, k1, g0, g1);
                            if (gcol < p.N && 8 * q + (lane & 7) < mrows)
                                *reinterpret_cast<uint4*>(yb + static_cast<size_t>(8 * q) * p.N) = out;
                        }
                    } else if (live) {
                        if (p.y_dt == TFP8B_F16) {
                            __half* yp = reinterpret_cast<__half*>(y0) + at0;
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (j < mrows) yp[static_cast<size_t>(j) * p.N] = __float2half_rn(val[j]);
                        } else if (p.y_dt == TFP8B_BF16) {
                            __nv_bfloat16* yp = reinterpret_cast<__nv_bfloat16*>(y0) + at0;
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (j < mrows) yp[static_cast<size_t>(j) * p.N] = __float2bfloat16_rn(val[j]);
                        } else {
                            float* yp = reinterpret_cast<float*>(y0) + at0;
#pragma unroll
                            for (int j = 0; j < 16; ++j) if (j < mrows) yp[static_cast<size_t>(j) * p.N] = val[j];
                        }
                    }
                } else if (OUT == GM_OUT_SPLITK) {
                    // this unit's share of the dot products, weight scale applied; the activation
                    // scale and the bias follow once all parts are in
                    float* w0 = p.ws + static_cast<size_t>(m0 + col) * p.N + n;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (live && j < mrows) atomicAdd(w0 + static_cast<size_t>(j) * p.N, val[j]);
                } else {
                    // a window of wider outputs: the local one only when the push warp serves the
                    // peers, else every destination element by element
                    const size_t at0 = static_cast<size_t>(m0 + col) * p.ldy + p.col0 + n;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (!live || j >= mrows) break;
                        const size_t at = at0 + static_cast<size_t>(j) * p.ldy;
                        if (OUT == GM_OUT_PUSH) {
                            store_dt(y0, at, val[j], p.y_dt);
                        } else {
#pragma unroll
                            for (int d = 0; d < GM_MAX_DST; ++d)
                                if (d < p.ndst) store_dt(p.y[d], at, val[j], p.y_dt);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (threadIdx.x == GM_EPI_WARP0 * 32) GM_TRACE(0, 253);
            if (lane == 0) {
                mbar_arrive(smem_u32(&hd->acc_empty[buf]));
                if (OUT == GM_OUT_PUSH) { __threadfence_block(); atomicAdd(&hd->tiles_stored, 1u); }   // this warp's part of the tile is in the local output
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
        if (lane == 0) GM_TRACE(0, 255);
    }
}

// ------------------------------------------------------------------ host side
static int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                       uint64_t outer, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    return encode_tensor_map(map, dt, 2, base, dims, strides, box, swz);
}

// SM count of a device, asked once per device (the query sits on the launch path of 50 us kernels).
static int device_sms(int dev) {
    static int cached[64] = {};
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    return sms;
}

template <int FMT, int OUT, int SC, int NG = 2>
static int launch_gemm_as(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, size_t smem, int dev, cudaStream_t st) {
    static unsigned long long configured = 0ull;             // one per instantiation: bit d = device d is set up
    if (dev >= 64 || !((configured >> dev) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<FMT, OUT, SC, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM_MAX);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm)");
        if (dev < 64) __atomic_fetch_or(&configured, 1ull << dev, __ATOMIC_RELAXED);
    }
    const int sms = device_sms(dev);
    const int grid = p.ntiles < sms ? p.ntiles : sms;
    gemm_kernel<FMT, OUT, SC, NG><<<grid, GM_THREADS, smem, st>>>(tw, tx, p);
    TFP8B_LAUNCH_CHECK("tfp8b_gemm");
    return TFP8B_OK;
}

template <int FMT>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, size_t smem, int dev, cudaStream_t st) {
    if (p.ng == 4) return p.ks > 1 ? launch_gemm_as<FMT, GM_OUT_SPLITK, 1, 4>(tw, tx, p, smem, dev, st)
                                   : launch_gemm_as<FMT, GM_OUT_PLAIN, 1, 4>(tw, tx, p, smem, dev, st);
    if (p.ks > 1) return p.sc_row > 0 ? launch_gemm_as<FMT, GM_OUT_SPLITK, 1>(tw, tx, p, smem, dev, st)
                                      : launch_gemm_as<FMT, GM_OUT_SPLITK, 0>(tw, tx, p, smem, dev, st);
    if (p.push) return launch_gemm_as<FMT, GM_OUT_PUSH, 0>(tw, tx, p, smem, dev, st);
    if (p.ndst > 1 || p.ldy != p.N || p.col0 != 0) return launch_gemm_as<FMT, GM_OUT_WINDOW, 0>(tw, tx, p, smem, dev, st);
    return p.sc_row > 0 ? launch_gemm_as<FMT, GM_OUT_PLAIN, 1>(tw, tx, p, smem, dev, st)
                        : launch_gemm_as<FMT, GM_OUT_PLAIN, 0>(tw, tx, p, smem, dev, st);
}

// ------------------------------------------------------------------ scratch for tfp8b_linear_static
// The tile GEMM consumes PREPARED activations (fp16 rows + one power-of-two scale per row), which
// the ordinary path keeps in a buffer the caller allocates. This array is that buffer for callers
// that have no way to allocate device memory; every GPU that loads the library carries it until
// the process exits. In host code its name is only a handle, not a device address: the address
// is fetched once per device with cudaGetSymbolAddress and handed to the kernels.
constexpr size_t STATIC_X16_ELEMS = 4u << 20;          // 4 Mi fp16 values = 8 MiB: M * K may not exceed this
constexpr int STATIC_MAX_ROWS = 8192;                  // row scales
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_X16_ELEMS * 2 + static_cast<size_t>(STATIC_MAX_ROWS) * 4;
static __device__ __align__(256) unsigned char g_linear_scratch[STATIC_SCRATCH_BYTES];

// Device address of the scratch array on the current device (looked up on first use per device).
static int static_scratch(unsigned char** out) {
    static unsigned char* ptrs[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) { set_error("tfp8b_linear_static: device index %d not supported", dev); return TFP8B_ERR_UNSUPPORTED; }
    unsigned char* p = __atomic_load_n(&ptrs[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_linear_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(linear scratch)");
        __atomic_store_n(&ptrs[dev], p, __ATOMIC_RELEASE);
    }
    *out = p;
    return TFP8B_OK;
}

int gemm_status(unsigned int* out, cudaStream_t st) {
    unsigned int* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&word), g_status);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(gemm status)");
    return read_and_clear_status(word, out, st);
}

}  // namespace tfp8b

using namespace tfp8b;

extern "C" int tfp8b_gemm(const void* x16, const float* xs, const uint8_t* codes, const void* scale, int scale_kind,
                          const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                          tfp8b_stream_t stream) {
    void* dst[1] = {y};
    return tfp8b_gemm_scatter(x16, xs, codes, scale, scale_kind, bias, dst, 1, N, 0, y_dtype, M, N, K, G, fmt, stream);
}

static int gemm_impl(const void* x16, const float* xs, const uint8_t* codes, const void* scale, int scale_kind,
                     const float* bias, void* const* y_dst, int n_dst, long long ldy, long long col0, int y_dtype,
                     int M, int N, int K, int G, int fmt, float* workspace, long long workspace_floats, tfp8b_stream_t stream);

extern "C" int tfp8b_gemm_scatter(const void* x16, const float* xs, const uint8_t* codes, const void* scale, int scale_kind,
                                  const float* bias, void* const* y_dst, int n_dst, long long ldy, long long col0, int y_dtype,
                                  int M, int N, int K, int G, int fmt, tfp8b_stream_t stream) {
    return gemm_impl(x16, xs, codes, scale, scale_kind, bias, y_dst, n_dst, ldy, col0, y_dtype, M, N, K, G, fmt, nullptr, 0, stream);
}

extern "C" int tfp8b_gemm_splitk(const void* x16, const float* xs, const uint8_t* codes, const void* scale, int scale_kind,
                                 const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt, float* workspace,
                                 long long workspace_floats, tfp8b_stream_t stream) {
    void* dst[1] = {y};
    return gemm_impl(x16, xs, codes, scale, scale_kind, bias, dst, 1, N, 0, y_dtype, M, N, K, G, fmt, workspace, workspace_floats, stream);
}

static int gemm_impl(const void* x16, const float* xs, const uint8_t* codes, const void* scale, int scale_kind,
                     const float* bias, void* const* y_dst, int n_dst, long long ldy, long long col0, int y_dtype,
                     int M, int N, int K, int G, int fmt, float* workspace, long long workspace_floats, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(M >= 0 && N >= 0 && K > 0 && G > 0, TFP8B_ERR_INVALID, "tfp8b_gemm: bad size M=%d N=%d K=%d G=%d", M, N, K, G);
    TFP8B_REQUIRE(y_dtype >= 0 && y_dtype <= 2, TFP8B_ERR_INVALID, "tfp8b_gemm: bad dtype");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_gemm: bad fmt %d", fmt);
    TFP8B_REQUIRE(scale_kind == TFP8B_SCALE_F32 || scale_kind == TFP8B_SCALE_UE8M0, TFP8B_ERR_INVALID,
                  "tfp8b_gemm: bad scale_kind %d", scale_kind);
    TFP8B_REQUIRE(y_dst && n_dst >= 1 && n_dst <= GM_MAX_DST, TFP8B_ERR_INVALID, "tfp8b_gemm: 1..%d output buffers, got %d",
                  GM_MAX_DST, n_dst);
    TFP8B_REQUIRE(col0 >= 0 && ldy >= col0 + N, TFP8B_ERR_INVALID,
                  "tfp8b_gemm: columns [%lld, %lld) do not fit a row pitch of %lld", col0, col0 + N, ldy);
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x16 && xs && codes && scale, TFP8B_ERR_INVALID, "tfp8b_gemm: null pointer");
    for (int d = 0; d < n_dst; ++d) TFP8B_REQUIRE(y_dst[d], TFP8B_ERR_INVALID, "tfp8b_gemm: null output pointer %d", d);
    TFP8B_REQUIRE(K % 32 == 0 && G % 32 == 0 && K % G == 0, TFP8B_ERR_UNSUPPORTED,
                  "tfp8b_gemm: need K %% 32 == 0, G %% 32 == 0, K %% G == 0 (K=%d G=%d)", K, G);
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(x16) | reinterpret_cast<uintptr_t>(codes)) & 15u) == 0, TFP8B_ERR_INVALID,
                  "tfp8b_gemm: x16 and codes must be 16-byte aligned");
    GemmParams p;
    p.xs = xs; p.scale = scale; p.bias = bias;
    for (int d = 0; d < GM_MAX_DST; ++d) p.y[d] = d < n_dst ? y_dst[d] : nullptr;
    p.ndst = n_dst; p.ldy = ldy; p.col0 = col0;
    // whole 16-byte chunks and 16-byte aligned rows everywhere: the push warp serves the peers
    {
        const long long esz = y_dtype == TFP8B_F32 ? 4 : 2;
        bool aligned = (ldy * esz) % 16 == 0 && (col0 * esz) % 16 == 0 && (static_cast<long long>(N) * esz) % 16 == 0;
        for (int d = 0; d < n_dst; ++d) aligned = aligned && (reinterpret_cast<uintptr_t>(y_dst[d]) & 15u) == 0;
        // TFP8B_GEMM_PUSH=0 in the environment falls back to element-wise peer stores from the epilogue
        static const int use_push = [] { const char* v = getenv("TFP8B_GEMM_PUSH"); return !(v && v[0] == '0'); }();
        p.push = (use_push && n_dst > 1 && aligned) ? 1 : 0;
    }
    p.M = M; p.N = N; p.K = K; p.G = G; p.scale_kind = scale_kind; p.y_dt = y_dtype;
    int bn = 16;
    while (bn < M && bn < 256) bn <<= 1;
    p.BN = bn;
    const int nkb = (K + GM_BK - 1) / GM_BK;
    // Two issuing threads, each with a double-buffered accumulator, while tensor memory has the
    // room: 2 x 2 x BN <= 512 columns. (Two threads accumulating into ONE accumulator is not an
    // option: that variant ended every BN = 256 launch with a launch failure.)
    p.m_tiles = (M + bn - 1) / bn;
    p.ntiles = p.m_tiles * ((N + GM_BM - 1) / GM_BM);
    p.rb = K % 128 == 0 ? 2 : 1;
    // Split-K (one activation tile, a workspace given): a CTA's k-loop is serial, about 0.3 us per
    // k-block whatever the tile width, so with few tiles of a long K the busiest CTA sets the time
    // (64 tiles of K = 8192 on 148 SMs: 84 SMs idle). Every tile is cut into ks units along K; the
    // units add their partial tiles into the FP32 workspace (atomics, L2 resident) and a final pass
    // applies the activation scale and the bias. The cost model counts k-blocks on the busiest CTA
    // plus a fixed turn-over per unit; it splits only where that clearly pays (fewer tiles than
    // half the SMs and a long K).
    p.ks = 1; p.nkbu = nkb; p.ws = nullptr;
    p.span = 0; p.span_total = 0; p.nkbt = nkb;
    int dev = 0;
    {
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    }
    const int sms = device_sms(dev);
    static const int use_splitk = [] { const char* v = getenv("TFP8B_GEMM_SPLITK"); return !(v && v[0] == '0'); }();
    if (use_splitk && workspace && n_dst == 1 && p.m_tiles == 1 && workspace_floats >= static_cast<long long>(M) * N) {
        // measured on B200: a unit costs about 8 k-blocks of turn-over (scale scan, pipeline fill
        // and drain, atomics), and the extra memset + final pass about 16
        constexpr int TURNOVER = 8, EXTRA_PASSES = 16;
        auto cost = [&](int ks) { return ((p.ntiles * ks + sms - 1) / sms) * (nkb / ks + TURNOVER) + (ks > 1 ? EXTRA_PASSES : 0); };
        int best = 1;
        for (int ks = 2; ks <= 16; ks <<= 1)
            if (nkb % ks == 0 && nkb / ks >= 8 && (p.rb == 1 || (nkb / ks) % 2 == 0) && cost(ks) < cost(best) &&
                cost(ks) * 6 < cost(1) * 5)                     // only for a clear gain: the split costs determinism
                best = ks;
        if (best > 1) { p.ks = best; p.nkbu = nkb / best; p.ws = workspace; p.ntiles *= best; }
        // At least one tile per SM, but a tile count that fills the last round badly (224 tiles on
        // 148 SMs: two rounds, the second half empty): split by spans instead. The k-blocks of all
        // tiles, tile after tile, are dealt out in equal contiguous spans, one per SM; a span is at
        // least one tile long, so a tile gets its sum from at most two CTAs and the result does not
        // depend on which of them adds first. Span ends are even: raw slots hold k-block pairs,
        // and two issuing threads take alternate k-blocks.
        static const int use_spans = [] { const char* v = getenv("TFP8B_GEMM_SPANS"); return !(v && v[0] == '0'); }();
        if (use_spans && best == 1 && p.ntiles >= sms && nkb % 2 == 0 && K % GM_BK == 0) {
            const long long total = static_cast<long long>(p.ntiles) * nkb;
            long long span = (total + sms - 1) / sms;
            span += span & 1;
            const long long rounds = (p.ntiles + sms - 1) / sms;
            // a span costs its k-blocks, two more turn-overs than a whole tile and the two extra passes
            if (total < (1ll << 30) && span >= nkb && (span + 2 * TURNOVER + EXTRA_PASSES) * 20 < rounds * nkb * 19) {
                p.span = static_cast<int>(span); p.span_total = static_cast<int>(total); p.nkbt = nkb;
                p.ks = 2;                                    // marks the split forms below: workspace, final pass
                p.ws = workspace;
                p.ntiles = static_cast<int>((total + span - 1) / span);   // = CTAs
            }
        }
    }
    p.nmma = (bn <= 128 && p.nkbu >= 4) ? 2 : 1;
    p.tmem_cols = 2 * p.nmma * bn < 32 ? 32 : 2 * p.nmma * bn;
    if (p.nmma != 1) p.push = 0;                             // warp 3 issues MMAs there
    // Shared memory: four decoded tiles (the groups' tiles in decode, the one in the MMA, one
    // spare); an activation ring as deep as pays (narrow tiles are paced by the L2 round trip of
    // their activation tile unless enough of them are in flight; at BN = 256 the MMA of a k-block
    // outlasts it); the rest raw codes -- the ring whose depth hides HBM latency. (At BN = 256 that
    // rest is two slots, four k-blocks: there the CTAs of the other activation tiles pull the
    // same stripe through L2.) Every ring's length is a multiple of the stride its users walk it
    // with (decode groups, issuing threads), so a slot is always revisited by the same user, in
    // order: a parity wait can then never be answered by a phase two completions away.
    p.x_bytes = bn * GM_BK * 2;
    const int budget = GM_SMEM_MAX - 1024 - GM_HEADER;
    // TFP8B_GEMM_NS=<4|6|8> overrides the number of decoded-tile slots (tuning).
    static const int ns_env = [] { const char* v = getenv("TFP8B_GEMM_NS"); return v ? atoi(v) : 0; }();
    const int raw_slot = p.rb * GM_RAW_BYTES;
    // K-group scales of a tile in shared memory (two tiles' worth), where a row's scales are whole
    // 16-byte pieces of at most 128 bytes: see the decode warps. TFP8B_GEMM_SCALE_CACHE=0 turns it off.
    int sc_row_wanted = 0;
    {
        static const int use_cache = [] { const char* v = getenv("TFP8B_GEMM_SCALE_CACHE"); return !(v && v[0] == '0'); }();
        const int row_bytes = (K / G) * (scale_kind == TFP8B_SCALE_UE8M0 ? 1 : 4);
        const bool plain_form = n_dst == 1 && ldy == N && col0 == 0;           // the other output forms keep the global path
        sc_row_wanted = (use_cache && plain_form && G != K && row_bytes % 16 == 0 && row_bytes <= 128 &&
                         (reinterpret_cast<uintptr_t>(scale) & 15u) == 0) ? row_bytes : 0;
    }
    // Ring sizes for `ng` decode groups; false if the raw ring would be shorter than its users need.
    auto size_rings = [&](int ng) {
        p.ng = ng;
        p.ns = (ns_env == 4 || ns_env == 6 || ns_env == 8) && ns_env % ng == 0 ? ns_env : 2 * ng;     // a multiple of the groups and of the issuing threads
        p.nx = bn >= 256 ? 4 : (bn == 128 ? 6 : GM_MAX_XSLOTS);      // even: two issuing threads walk it with stride 2
        if (p.ns > 4 && bn >= 32) p.nx = 4;
        const int raw_stride = ng / p.rb;                             // slots between a group's consecutive k-blocks
        const int min_raw = raw_stride > 2 ? raw_stride : 2;
        p.sc_row = sc_row_wanted;
        if ((budget - p.ns * GM_A_BYTES - p.nx * p.x_bytes - 2 * GM_BM * p.sc_row) / raw_slot < min_raw) p.sc_row = 0;   // no room at this tile width
        p.sr = (budget - p.ns * GM_A_BYTES - p.nx * p.x_bytes - 2 * GM_BM * p.sc_row) / raw_slot;
        if (p.sr > GM_MAX_SLOTS) p.sr = GM_MAX_SLOTS;
        p.sr -= p.sr % raw_stride;
        return p.sr >= raw_stride && p.sr >= 2;
    };
    // Four groups where they pay (measured, 28672 x 8192 with 128-wide groups: 98 -> 92 us at 16 rows,
    // 101 -> 95 at 32; 14336 x 4096 at 24 rows: 35 -> 31; units of 32 k-blocks: 7 % slower): narrow
    // tiles, scales cached, plain or split-K output, units of at least 64 k-blocks, and at least
    // four raw slots left. TFP8B_GEMM_GROUPS=2 turns it off.
    static const int groups_env = [] { const char* v = getenv("TFP8B_GEMM_GROUPS"); return v ? atoi(v) : 0; }();
    bool four = groups_env != 2 && bn <= 32 && p.nkbu >= 64 && sc_row_wanted > 0 && p.push == 0 && n_dst == 1 && size_rings(4) &&
                p.sc_row > 0 && p.sr >= 4;
    if (!four) TFP8B_REQUIRE(size_rings(2), TFP8B_ERR_INVALID, "tfp8b_gemm: ring sizes ns=%d nx=%d sr=%d do not fit", p.ns, p.nx, p.sr);
    const int sc_bytes = 2 * GM_BM * p.sc_row;
    const size_t smem = 1024 + GM_HEADER + static_cast<size_t>(p.ns) * GM_A_BYTES + static_cast<size_t>(p.nx) * p.x_bytes +
                        static_cast<size_t>(p.sr) * raw_slot + sc_bytes;

    CUtensorMap tw, tx;
    int rc;
    if (p.rb == 2) {
        // codes seen as [K/128][N][128 bytes]: one copy brings 128 rows x 128 contiguous bytes
        const cuuint64_t wd[3] = {128, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K / 128)};
        const cuuint64_t ws[2] = {static_cast<cuuint64_t>(K), 128};
        const cuuint32_t wb[3] = {128, GM_BM, 1};
        // 128-byte swizzle: the 16-byte chunk index of a row is XORed with (row & 7), which lets
        // the decode warps read 8 rows' chunks without two of them sharing a bank
        rc = encode_tensor_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, codes, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        rc = make_map_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, static_cast<uint64_t>(K), static_cast<uint64_t>(N),
                         GM_BK, GM_BM, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    if (rc != TFP8B_OK) return rc;
    rc = make_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                     GM_BK, static_cast<uint32_t>(bn), CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TFP8B_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p.ks > 1) {
        cudaError_t e = cudaMemsetAsync(workspace, 0, static_cast<size_t>(M) * N * sizeof(float), st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(split-K workspace)");
    }
    rc = fmt == TFP8B_E4M3FN ? launch_gemm<TFP8B_E4M3FN>(tw, tx, p, smem, dev, st) : launch_gemm<TFP8B_E5M2>(tw, tx, p, smem, dev, st);
    if (rc != TFP8B_OK || p.ks == 1) return rc;
    // y = workspace * xs[m] + bias[n], rounded once to the output type
    return tfp8b_epilogue(workspace, xs, bias, y_dst[0], y_dtype, M, N, static_cast<int>(ldy), stream);
}

extern "C" int tfp8b_linear_static(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
                                   const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                                   tfp8b_stream_t stream) {
    TFP8B_REQUIRE(M >= 0 && N >= 0 && K > 0, TFP8B_ERR_INVALID, "tfp8b_linear_static: bad size M=%d N=%d K=%d", M, N, K);
    TFP8B_REQUIRE(M <= STATIC_MAX_ROWS && static_cast<size_t>(M) * static_cast<size_t>(K) <= STATIC_X16_ELEMS,
                  TFP8B_ERR_UNSUPPORTED,
                  "tfp8b_linear_static: M=%d x K=%d exceeds the built-in scratch (at most %d rows and %zu activation "
                  "values per call); use tfp8b_prep + tfp8b_gemm with a buffer of your own", M, K, STATIC_MAX_ROWS,
                  STATIC_X16_ELEMS);
    if (M == 0 || N == 0) return TFP8B_OK;
    unsigned char* scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc != TFP8B_OK) return rc;
    void* x16 = scratch;
    float* xs = reinterpret_cast<float*>(scratch + STATIC_X16_ELEMS * 2);
    // prep overwrites every value the GEMM will read (M * K activations, M scales): nothing in the
    // array has to start out as zero, whatever an earlier call left there.
    rc = tfp8b_prep(x, x_dtype, x16, xs, M, K, stream);
    if (rc != TFP8B_OK) return rc;
    return tfp8b_gemm(x16, xs, codes, scale, scale_kind, bias, y, y_dtype, M, N, K, G, fmt, stream);
}
