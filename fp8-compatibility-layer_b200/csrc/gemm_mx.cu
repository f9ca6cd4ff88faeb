// W8A8 GEMM: FP8 activations x FP8 weights, both as codes straight into the tensor cores.
//
//   y[m,n] = sum_kb ( sum_{k in kb} dec(a[m,k]) * dec(w[n,k]) ) * sa[m,kb] * sw[n,kb] + bias[n]      (block mode)
//   y[m,n] = ( sum_k dec(a[m,k]) * dec(w[n,k]) ) * sa[m] * sw[n] + bias[n]                            (row/col mode)
//
// kb runs over 32-wide blocks of K. This is the B200 form of the reference project's other native
// kernel (fp8_gemm_kernel.cu there: a table decode to fp16, WMMA per 32-wide block, scales applied
// to each block's partial product in FP32 registers). Here nothing is decoded:
//   * block mode with UE8M0 scales is exactly what tcgen05.mma.kind::mxf8f6f4.block_scale computes:
//     the exponent bytes sit in tensor memory next to the accumulator and the tensor core applies
//     them per 32-wide block, so the kernel is a plain TMA -> MMA pipeline;
//   * row/col mode is tcgen05.mma.kind::f8f6f4 over the whole K, the two scales applied in the
//     epilogue (FP32 or UE8M0);
//   * block mode with FP32 scales cannot be given to the tensor core (it only takes exponents).
//     It runs the same MMAs one 32-wide block at a time into a fresh accumulator, and the epilogue
//     warps scale each block's partial product and add it up in registers -- the reference's own
//     scheme, and as in the reference far slower than the other three forms.
// Both operands are K-major ([M, K] and [N, K] row-major codes), E4M3FN or E5M2 independently.
//
// One CTA per SM walks 128 x 128 output tiles (the activation-row tile is the fast index, so CTAs
// that run together share a weight stripe through L2). Warp 0 is the TMA producer: per 128-wide
// k-tile one 16 KB tile of each operand in the 128-byte swizzle plus, in MX mode, the two 512-byte
// scale chunks of the tile; warp 1 copies the scale chunks into tensor memory (tcgen05.cp) and
// issues four MMAs (K = 32 each) per k-tile; warps 4..7 drain the FP32 accumulator (two buffers:
// a tile's epilogue overlaps the next tile's main loop), add the bias and store rows.
//
// Scale layout of the MX mode ("packed"): for every 128 rows x 128 K (4 blocks) one 512-byte chunk
// with the byte of (row r, block b) at (r % 32) * 16 + (r / 32) * 4 + b, chunks ordered
// [row tile][k tile]. That is the order tcgen05.cp.32x128b.warpx4 turns into the 4 tensor-memory
// columns the MMA reads its scales from; tfp8b_mx_pack_scales produces it from the row-major
// [rows, K/32] bytes, and the activation quantizer can write it directly.
// Every mbarrier wait is bounded (status bit + the thread keeps walking its loops).
#include <stdlib.h>

#include "common.cuh"

namespace tfp8b {

constexpr int MX_BM = 128, MX_BK = 128;
constexpr int MX_MAX_STAGES = 6;
constexpr int MX_THREADS = 256;                         // warp 0 producer, warp 1 MMA, warps 4..7 epilogue
constexpr int MX_A_BYTES = MX_BM * MX_BK;               // 16 KB of activation codes per stage
constexpr int MX_SF_BYTES = 512;                        // one scale chunk: 128 rows x 4 blocks
constexpr int MX_HEADER = 1024;
constexpr int MX_TMEM_COLS = 512;
// Per tile width BN (weight rows per tile = accumulator columns). 192 is the widest that leaves
// room in tensor memory for two accumulators AND the scale columns (2 x 192 + 5 x 12 = 444 of 512
// columns; with 256 the two accumulators alone take all 512): the wider the tile, the fewer bytes
// cross from L2 per FLOP, and that crossing is what bounds this kernel. A 192-row tile starts at a
// multiple of 64 rows, so it reads two 128-row scale chunks and its scale columns begin at column
// 0 or 2 of the first chunk.
template <int BN>
struct MxCfg {
    static constexpr int B_BYTES = BN * MX_BK;
    static constexpr int SFB_CHUNKS = BN > 128 ? 2 : 1;
    static constexpr int STAGE_BYTES = (MX_A_BYTES + B_BYTES + MX_SF_BYTES * (1 + SFB_CHUNKS) + 1023) / 1024 * 1024;
    static constexpr int STAGES = BN > 128 ? 5 : 6;
    static constexpr int SMEM = 1024 + MX_HEADER + STAGES * STAGE_BYTES;
    static constexpr int SF_COLS = 4 + 4 * SFB_CHUNKS;       // tensor-memory columns of one stage's scales
    static constexpr int SF_COL0 = 2 * BN;
    static_assert(SF_COL0 + SF_COLS * STAGES <= MX_TMEM_COLS, "tensor memory: accumulators + scale columns");
    static_assert(SMEM <= 232448 && STAGES <= MX_MAX_STAGES, "shared memory");
};

constexpr int MXM_BLOCK_E8 = 0, MXM_ROWCOL = 1, MXM_BLOCK_F32 = 2;

struct MxParams {
    const uint8_t* sfa;       // MX: packed UE8M0 chunks of the activations; block-f32: float [M, K/32]; row/col: [M] f32 or u8
    const uint8_t* sfw;       // the same for the weights ([N, ...])
    const float* bias;
    void* y;
    int M, N, K, y_dt, a_fmt, w_fmt, scale_kind;
    int m_tiles, ntiles, nkt, n_chunks;     // n_chunks: 128-row scale chunks of the weight
};

struct MxHeader {
    uint64_t full[MX_MAX_STAGES], empty[MX_MAX_STAGES];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
};
static_assert(sizeof(MxHeader) <= MX_HEADER, "header too large");

// ------------------------------------------------------------------ tcgen05 wrappers (this file's own)
__device__ __forceinline__ void mx_tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mx_tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void mx_tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mx_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mx_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mx_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem] with per-32-block UE8M0 scales read from tensor memory
__device__ __forceinline__ void mx_mma_block_scaled(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                    uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
__device__ __forceinline__ void mx_mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 tensor-memory columns, the same 32 lanes in all four lane quarters
__device__ __forceinline__ void mx_cp_sf(uint32_t tmem_dst, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc) : "memory");
}
__device__ __forceinline__ void mx_tmem_ld16(uint32_t taddr, uint32_t r[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void mx_tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in the 128-byte swizzle (rows of 128 bytes, 8-row groups 1024 bytes apart);
// stepping K by 32 one-byte elements advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t mx_desc_sw128(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// A 512-byte scale chunk: 32 rows of 16 bytes, no swizzle (8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t mx_desc_sf(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) | (8ull << 16) | (8ull << 32) | (1ull << 46);
}

__device__ __forceinline__ float mx_scale(const void* s, size_t i, int kind) { return load_scale(s, i, kind); }

// ------------------------------------------------------------------ the kernel
template <int MODE, int BN>
__global__ void __launch_bounds__(MX_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const MxParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    MxHeader* hd = reinterpret_cast<MxHeader*>(smem);
    uint8_t* stages = smem + MX_HEADER;
    using C = MxCfg<BN>;
    constexpr int MX_BN = BN, MX_STAGES = C::STAGES, MX_STAGE_BYTES = C::STAGE_BYTES;
    constexpr int OFF_B = MX_A_BYTES, OFF_SFA = MX_A_BYTES + C::B_BYTES, OFF_SFB = OFF_SFA + MX_SF_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int my_tiles = (p.ntiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    auto tile_of = [&](int i) { return static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x); };
    auto tile_m0 = [&](int i) { return (tile_of(i) % p.m_tiles) * MX_BM; };
    auto tile_n0 = [&](int i) { return (tile_of(i) / p.m_tiles) * MX_BN; };
    // block mode with FP32 scales: every 32-wide block is an accumulator hand-over of its own
    constexpr bool PER_BLOCK = MODE == MXM_BLOCK_F32;
    const int units_per_tile = PER_BLOCK ? p.nkt * 4 : 1;      // accumulator hand-overs per output tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < MX_STAGES; ++s) {
            mbar_init(smem_u32(&hd->full[s]), 1);
            mbar_init(smem_u32(&hd->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&hd->acc_full[b]), 1);
            mbar_init(smem_u32(&hd->acc_empty[b]), 4);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_w);
    }
    if (warp == 1) {
        mx_tmem_alloc(smem_u32(&hd->tmem_base), MX_TMEM_COLS);
        mx_tmem_relinquish();
    }
    mx_fence_before();
    __syncthreads();
    mx_fence_after();
    const uint32_t tmem_base = hd->tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            const uint64_t pol_a = l2_policy_evict_last(), pol_w = p.m_tiles == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
            int slot = 0;
            uint32_t phase = 1;
            bool ok = true, first_pass = true;
            for (int i = 0; i < my_tiles && ok; ++i) {
                const int m0 = tile_m0(i), n0 = tile_n0(i);
                // the weight tile's scale chunks: one, or two for a 192-row tile (the second may lie
                // beyond the last chunk of the weight: then it is not fetched, its columns are unused)
                const int c0 = n0 / 128;
                const bool two = C::SFB_CHUNKS == 2 && c0 + 1 < p.n_chunks;
                const uint32_t tx = MX_A_BYTES + C::B_BYTES + (MODE == MXM_BLOCK_E8 ? MX_SF_BYTES * (two ? 3u : 2u) : 0u);
                for (int kt = 0; kt < p.nkt; ++kt) {
                    if (!first_pass && !mbar_wait(smem_u32(&hd->empty[slot]), phase, STATUS_GEMM_WAIT)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&hd->full[slot]);
                    uint8_t* st = stages + static_cast<size_t>(slot) * MX_STAGE_BYTES;
                    mbar_expect_tx(bar, tx);
                    tma_load_2d(smem_u32(st), &tm_a, kt * MX_BK, m0, bar, pol_a);
                    tma_load_2d(smem_u32(st + OFF_B), &tm_w, kt * MX_BK, n0, bar, pol_w);
                    if (MODE == MXM_BLOCK_E8) {
                        bulk_g2s(smem_u32(st + OFF_SFA), p.sfa + (static_cast<size_t>(m0 / MX_BM) * p.nkt + kt) * MX_SF_BYTES,
                                 MX_SF_BYTES, bar, pol_a);
                        bulk_g2s(smem_u32(st + OFF_SFB), p.sfw + (static_cast<size_t>(c0) * p.nkt + kt) * MX_SF_BYTES, MX_SF_BYTES, bar, pol_w);
                        if (two)
                            bulk_g2s(smem_u32(st + OFF_SFB + MX_SF_BYTES), p.sfw + (static_cast<size_t>(c0 + 1) * p.nkt + kt) * MX_SF_BYTES,
                                     MX_SF_BYTES, bar, pol_w);
                    }
                    if (++slot == MX_STAGES) { slot = 0; phase ^= 1u; first_pass = false; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // A = activations (M = 128 rows), B = weights (N = 128 rows), both K-major, D fp32
            const uint32_t shape = (static_cast<uint32_t>(MX_BN >> 3) << 17) | (static_cast<uint32_t>(MX_BM >> 4) << 24);
            const uint32_t fmts = (static_cast<uint32_t>(p.a_fmt) << 7) | (static_cast<uint32_t>(p.w_fmt) << 10);
            const uint32_t idesc_mx = shape | fmts | (1u << 23);                  // scale format E8M0
            const uint32_t idesc_f8 = shape | fmts | (1u << 4);                   // D format F32
            int slot = 0;
            uint32_t phase = 0;
            bool ok = true;
            int unit = 0;                               // accumulator hand-overs of this CTA so far
            for (int i = 0; i < my_tiles && ok; ++i) {
                uint32_t accumulate = 0u;
                uint32_t tmem_acc = 0u;
                auto begin_unit = [&]() {
                    const int buf = unit & 1;
                    if (unit >= 2) ok = mbar_wait(smem_u32(&hd->acc_empty[buf]), ((unit >> 1) - 1) & 1, STATUS_GEMM_WAIT);
                    mx_fence_after();
                    tmem_acc = tmem_base + static_cast<uint32_t>(buf * MX_BN);
                };
                auto end_unit = [&]() {
                    if (ok) mx_commit(smem_u32(&hd->acc_full[unit & 1]));
                    ++unit;
                };
                if (!PER_BLOCK) begin_unit();
                for (int kt = 0; kt < p.nkt && ok; ++kt) {
                    ok = mbar_wait(smem_u32(&hd->full[slot]), phase, STATUS_GEMM_WAIT);
                    if (!ok) break;
                    mx_fence_after();
                    const uint32_t st = smem_u32(stages + static_cast<size_t>(slot) * MX_STAGE_BYTES);
                    const uint64_t da = mx_desc_sw128(st), db = mx_desc_sw128(st + OFF_B);
                    if (MODE == MXM_BLOCK_E8) {
                        const uint32_t tsfa = tmem_base + static_cast<uint32_t>(C::SF_COL0 + slot * C::SF_COLS);
                        mx_cp_sf(tsfa, mx_desc_sf(st + OFF_SFA));
                        mx_cp_sf(tsfa + 4u, mx_desc_sf(st + OFF_SFB));
                        if (C::SFB_CHUNKS == 2) mx_cp_sf(tsfa + 8u, mx_desc_sf(st + OFF_SFB + MX_SF_BYTES));
                        // the tile's first weight row inside its first chunk: 32 rows per scale column
                        const uint32_t tsfb = tsfa + 4u + static_cast<uint32_t>((tile_n0(i) & 127) >> 5);
#pragma unroll
                        for (uint32_t kb = 0; kb < 4; ++kb) {
                            // block kb of the k-tile: byte kb of the scale columns, for both operands
                            mx_mma_block_scaled(tmem_acc, da + 2 * kb, db + 2 * kb, idesc_mx | (kb << 4) | (kb << 29), tsfa, tsfb, accumulate);
                            accumulate = 1u;
                        }
                    } else if (MODE == MXM_ROWCOL) {
#pragma unroll
                        for (uint32_t kb = 0; kb < 4; ++kb) {
                            mx_mma_f8(tmem_acc, da + 2 * kb, db + 2 * kb, idesc_f8, accumulate);
                            accumulate = 1u;
                        }
                    } else {
                        for (uint32_t kb = 0; kb < 4 && ok; ++kb) {              // one block, one accumulator hand-over
                            begin_unit();
                            if (!ok) break;
                            mx_mma_f8(tmem_acc, da + 2 * kb, db + 2 * kb, idesc_f8, 0u);
                            end_unit();
                        }
                    }
                    if (ok) mx_commit(smem_u32(&hd->empty[slot]));
                    if (++slot == MX_STAGES) { slot = 0; phase ^= 1u; }
                }
                if (!PER_BLOCK) end_unit();
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- epilogue warps
        const int quarter = warp & 3;
        bool ok = true;
        int unit = 0;
        for (int i = 0; i < my_tiles; ++i) {
            const int m0 = tile_m0(i), n0 = tile_n0(i);
            const int m = m0 + quarter * 32 + lane;
            const bool row_live = m < p.M;
            float acc[PER_BLOCK ? MX_BN : 1];
            if (PER_BLOCK) {
#pragma unroll
                for (int c = 0; c < (PER_BLOCK ? MX_BN : 1); ++c) acc[c] = 0.f;
            }
            const float sa_row = (MODE == MXM_ROWCOL && row_live) ? mx_scale(p.sfa, m, p.scale_kind) : 1.f;
            for (int u = 0; u < units_per_tile; ++u, ++unit) {
                const int buf = unit & 1;
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->acc_full[buf]), (unit >> 1) & 1, STATUS_GEMM_WAIT));
                if (!ok) continue;
                mx_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * MX_BN);
                // block mode with FP32 scales: this hand-over is block u of K; its partial product is
                // scaled by sa[m, u] * sw[n, u] and added up here, in FP32 registers
                const int nblk = p.K / 32;
                const float sa_blk = (PER_BLOCK && row_live) ? reinterpret_cast<const float*>(p.sfa)[static_cast<size_t>(m) * nblk + u] : 0.f;
#pragma unroll
                for (int col = 0; col < MX_BN; col += 16) {
                    uint32_t v[16];
                    mx_tmem_ld16(taddr + col, v);
                    mx_tmem_ld_wait();
                    if (PER_BLOCK) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int n = n0 + col + j;
                            const float sw = n < p.N ? __ldg(reinterpret_cast<const float*>(p.sfw) + static_cast<size_t>(n) * nblk + u) : 0.f;
                            acc[PER_BLOCK ? col + j : 0] = fmaf(__uint_as_float(v[j]), sa_blk * sw, acc[PER_BLOCK ? col + j : 0]);
                        }
                    } else {
                        float out[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int n = n0 + col + j;
                            float val = __uint_as_float(v[j]);
                            if (MODE == MXM_ROWCOL) val *= sa_row * (n < p.N ? mx_scale(p.sfw, n, p.scale_kind) : 0.f);
                            out[j] = val + ((p.bias && n < p.N) ? __ldg(p.bias + n) : 0.f);
                        }
                        if (row_live) {
                            const size_t at = static_cast<size_t>(m) * p.N + n0 + col;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (n0 + col + j < p.N) store_dt(p.y, at + j, out[j], p.y_dt);
                        }
                    }
                }
                mx_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&hd->acc_empty[buf]));
            }
            if (PER_BLOCK && ok && row_live) {
                const size_t at = static_cast<size_t>(m) * p.N + n0;
#pragma unroll
                for (int c = 0; c < (PER_BLOCK ? MX_BN : 1); ++c)
                    if (n0 + c < p.N) store_dt(p.y, at + c, acc[PER_BLOCK ? c : 0] + (p.bias ? __ldg(p.bias + n0 + c) : 0.f), p.y_dt);
            }
        }
    }
    mx_fence_before();
    __syncthreads();
    if (warp == 1) {
        mx_fence_after();
        mx_tmem_dealloc(tmem_base, MX_TMEM_COLS);
    }
}

// ------------------------------------------------------------------ scale packing and the activation quantizer
// dst: ceil(R/128) x ceil(KB/4) chunks of 512 bytes; padding rows / blocks get 127 (the scale 1).
__global__ void __launch_bounds__(256) mx_pack_scales_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                             int R, int KB, int RT, int KT) {
    const long long total = static_cast<long long>(RT) * KT * 128;            // one 32-bit word (4 blocks of one row) per item
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int w = static_cast<int>(i % 128);                                  // word inside the chunk: (r % 32) * 4 + (r % 128) / 32
        const long long chunk = i / 128;
        const int kt = static_cast<int>(chunk % KT), rt = static_cast<int>(chunk / KT);
        const int r = rt * 128 + (w & 3) * 32 + (w >> 2);
        uint32_t word = 0u;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int kb = kt * 4 + b;
            const uint32_t v = (r < R && kb < KB) ? src[static_cast<size_t>(r) * KB + kb] : 127u;
            word |= v << (8 * b);
        }
        reinterpret_cast<uint32_t*>(dst)[i] = word;
    }
}

// Activation / weight rows -> FP8 codes with one scale per 32-wide block of K, the reference's
// quantize_k (fp8_cuda.py:74-91 there):  s = max(amax / fmax, 1e-12);  UE8M0: e = clamp(ceil(log2 s),
// -127, 127), s = 2^e, byte e + 127;  codes = FP8(clamp(x / s, +-fmax)). One thread per block.
// layout 0: scales row-major [R, K/32]; 1: the packed chunk order above (UE8M0 only).
template <typename T, int FMT>
__global__ void __launch_bounds__(256) quantize_k_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, void* __restrict__ scale,
                                                         int R, int K, int ue8m0, int layout) {
    const int KB = K / 32;
    const long long total = static_cast<long long>(R) * KB;
    const float fmax = FMT == TFP8B_E4M3FN ? 448.f : 57344.f;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / KB), kb = static_cast<int>(i % KB);
        const T* src = x + static_cast<size_t>(r) * K + static_cast<size_t>(kb) * 32;
        float v[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = to_f32(src[t]);
        float amax = 0.f;
        bool has_nan = false;
#pragma unroll
        for (int t = 0; t < 32; ++t) { amax = fmaxf(amax, fabsf(v[t])); has_nan = has_nan || v[t] != v[t]; }
        float s = fmaxf(__fdiv_rn(amax, fmax), 1e-12f);
        if (has_nan) s = __uint_as_float(0x7FC00000u);                            // a NaN in the block: NaN scale, NaN codes (as torch's amax)
        uint32_t byte = 0u;
        if (ue8m0) {
            float e = ceilf(log2f(s));
            e = fminf(fmaxf(e, -127.f), 127.f);
            if (s != s) { byte = 255u; }
            else { byte = static_cast<uint32_t>(static_cast<int>(e) + 127); s = exp2f(e); }
        }
        uint32_t codes[8];
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            uint32_t word = 0u;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float t = __fdiv_rn(v[4 * w + b], s);
                if (t == t) t = fminf(fmaxf(t, -fmax), fmax);                     // a NaN quotient stays NaN (fminf / fmaxf would drop it)
                word |= encode1<FMT>(t, TFP8B_NAN_CAST) << (8 * b);
            }
            codes[w] = word;
        }
        uint4* dst = reinterpret_cast<uint4*>(q + static_cast<size_t>(r) * K + static_cast<size_t>(kb) * 32);
        dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
        dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
        if (!ue8m0) {
            reinterpret_cast<float*>(scale)[i] = s;
        } else if (layout == 0) {
            reinterpret_cast<uint8_t*>(scale)[i] = static_cast<uint8_t>(byte);
        } else {
            const int KT = (KB + 3) / 4;
            const size_t at = (static_cast<size_t>(r / 128) * KT + kb / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (kb & 3);
            reinterpret_cast<uint8_t*>(scale)[at] = static_cast<uint8_t>(byte);
        }
    }
}

static int mx_device_sms() {
    static int cached[64] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

template <int MODE, int BN>
static int launch_mx(const void* a_codes, const void* w_codes, MxParams p, cudaStream_t st) {
    using C = MxCfg<BN>;
    static unsigned long long configured = 0ull;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev >= 64 || !((configured >> dev) & 1ull)) {
        e = cudaFuncSetAttribute(gemm_mx_kernel<MODE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm_mx)");
        if (dev < 64) __atomic_fetch_or(&configured, 1ull << dev, __ATOMIC_RELAXED);
    }
    p.m_tiles = (p.M + MX_BM - 1) / MX_BM;
    p.ntiles = p.m_tiles * ((p.N + BN - 1) / BN);
    p.n_chunks = (p.N + 127) / 128;
    CUtensorMap ta, tw;
    {
        const cuuint64_t da[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
        const cuuint64_t dw[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.N)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.K)};
        const cuuint32_t box_a[2] = {MX_BK, MX_BM}, box_w[2] = {MX_BK, BN};
        int rc = encode_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a_codes, da, strides, box_a, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != TFP8B_OK) return rc;
        rc = encode_tensor_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w_codes, dw, strides, box_w, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != TFP8B_OK) return rc;
    }
    const int sms = mx_device_sms();
    gemm_mx_kernel<MODE, BN><<<p.ntiles < sms ? p.ntiles : sms, MX_THREADS, C::SMEM, st>>>(ta, tw, p);
    TFP8B_LAUNCH_CHECK("tfp8b_gemm_w8a8");
    return TFP8B_OK;
}

int gemm_mx_status(unsigned int* out, cudaStream_t st) {
    unsigned int* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&word), g_status);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(gemm_mx status)");
    return read_and_clear_status(word, out, st);
}

}  // namespace tfp8b

using namespace tfp8b;

extern "C" long long tfp8b_mx_packed_scale_bytes(int rows, int K) {
    if (rows < 0 || K < 0) return -1;
    const long long rt = (rows + 127) / 128, kt = (K / 32 + 3) / 4;
    return rt * kt * 512;
}

extern "C" int tfp8b_mx_pack_scales(const uint8_t* scale_rowmajor, uint8_t* packed, int rows, int K, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(rows >= 0 && K >= 0 && K % 32 == 0, TFP8B_ERR_INVALID, "tfp8b_mx_pack_scales: bad size rows=%d K=%d", rows, K);
    if (rows == 0 || K == 0) return TFP8B_OK;
    TFP8B_REQUIRE(scale_rowmajor && packed, TFP8B_ERR_INVALID, "tfp8b_mx_pack_scales: null pointer");
    TFP8B_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_mx_pack_scales: packed must be 16-byte aligned");
    const int KB = K / 32, RT = (rows + 127) / 128, KT = (KB + 3) / 4;
    const long long items = static_cast<long long>(RT) * KT * 128;
    const int grid = static_cast<int>(items / 256 + 1 > 148 * 8 ? 148 * 8 : items / 256 + 1);
    mx_pack_scales_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(scale_rowmajor, packed, rows, KB, RT, KT);
    TFP8B_LAUNCH_CHECK("tfp8b_mx_pack_scales");
    return TFP8B_OK;
}

extern "C" int tfp8b_quantize_k(const void* x, int x_dtype, uint8_t* codes, void* scale, int rows, int K, int fmt, int ue8m0,
                                int packed, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(rows >= 0 && K >= 0 && K % 32 == 0, TFP8B_ERR_INVALID, "tfp8b_quantize_k: need K %% 32 == 0 (rows=%d K=%d)", rows, K);
    TFP8B_REQUIRE(x_dtype >= 0 && x_dtype <= 2, TFP8B_ERR_INVALID, "tfp8b_quantize_k: bad dtype");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_quantize_k: bad fmt %d", fmt);
    TFP8B_REQUIRE(!packed || ue8m0, TFP8B_ERR_INVALID, "tfp8b_quantize_k: the packed scale layout holds UE8M0 bytes only");
    if (rows == 0 || K == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x && codes && scale, TFP8B_ERR_INVALID, "tfp8b_quantize_k: null pointer");
    TFP8B_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_quantize_k: codes must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (packed) {
        // padding rows / blocks of the chunks must hold a valid scale: fill with 127 (= 1.0) first
        cudaError_t e = cudaMemsetAsync(scale, 127, static_cast<size_t>(tfp8b_mx_packed_scale_bytes(rows, K)), st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(packed scales)");
    }
    const long long items = static_cast<long long>(rows) * (K / 32);
    const int grid = static_cast<int>((items + 255) / 256 > 148 * 16 ? 148 * 16 : (items + 255) / 256);
#define QK_CASE(T, DT, F) \
    if (x_dtype == DT && fmt == F) quantize_k_kernel<T, F><<<grid, 256, 0, st>>>(static_cast<const T*>(x), codes, scale, rows, K, ue8m0, packed)
    QK_CASE(__half, TFP8B_F16, TFP8B_E4M3FN); QK_CASE(__half, TFP8B_F16, TFP8B_E5M2);
    QK_CASE(__nv_bfloat16, TFP8B_BF16, TFP8B_E4M3FN); QK_CASE(__nv_bfloat16, TFP8B_BF16, TFP8B_E5M2);
    QK_CASE(float, TFP8B_F32, TFP8B_E4M3FN); QK_CASE(float, TFP8B_F32, TFP8B_E5M2);
#undef QK_CASE
    TFP8B_LAUNCH_CHECK("tfp8b_quantize_k");
    return TFP8B_OK;
}

extern "C" int tfp8b_gemm_w8a8(const uint8_t* a_codes, const void* a_scale, int a_fmt, const uint8_t* w_codes, const void* w_scale,
                               int w_fmt, int scale_mode, int scale_kind, const float* bias, void* y, int y_dtype, int M, int N, int K,
                               tfp8b_stream_t stream) {
    TFP8B_REQUIRE(M >= 0 && N >= 0 && K > 0, TFP8B_ERR_INVALID, "tfp8b_gemm_w8a8: bad size M=%d N=%d K=%d", M, N, K);
    TFP8B_REQUIRE(y_dtype >= 0 && y_dtype <= 2, TFP8B_ERR_INVALID, "tfp8b_gemm_w8a8: bad dtype");
    TFP8B_REQUIRE((a_fmt == TFP8B_E4M3FN || a_fmt == TFP8B_E5M2) && (w_fmt == TFP8B_E4M3FN || w_fmt == TFP8B_E5M2), TFP8B_ERR_INVALID,
                  "tfp8b_gemm_w8a8: bad fmt %d / %d", a_fmt, w_fmt);
    TFP8B_REQUIRE(scale_mode == TFP8B_W8A8_BLOCK32 || scale_mode == TFP8B_W8A8_ROWCOL, TFP8B_ERR_INVALID,
                  "tfp8b_gemm_w8a8: bad scale_mode %d", scale_mode);
    TFP8B_REQUIRE(scale_kind == TFP8B_SCALE_F32 || scale_kind == TFP8B_SCALE_UE8M0, TFP8B_ERR_INVALID,
                  "tfp8b_gemm_w8a8: bad scale_kind %d", scale_kind);
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(a_codes && a_scale && w_codes && w_scale && y, TFP8B_ERR_INVALID, "tfp8b_gemm_w8a8: null pointer");
    TFP8B_REQUIRE(K % 128 == 0, TFP8B_ERR_UNSUPPORTED, "tfp8b_gemm_w8a8: need K %% 128 == 0 (K=%d)", K);
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(a_codes) | reinterpret_cast<uintptr_t>(w_codes) | reinterpret_cast<uintptr_t>(a_scale) |
                    reinterpret_cast<uintptr_t>(w_scale)) & 15u) == 0, TFP8B_ERR_INVALID,
                  "tfp8b_gemm_w8a8: codes and scales must be 16-byte aligned");
    MxParams p;
    p.sfa = static_cast<const uint8_t*>(a_scale); p.sfw = static_cast<const uint8_t*>(w_scale);
    p.bias = bias; p.y = y;
    p.M = M; p.N = N; p.K = K; p.y_dt = y_dtype; p.a_fmt = a_fmt; p.w_fmt = w_fmt; p.scale_kind = scale_kind;
    p.nkt = K / MX_BK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // TFP8B_W8A8_BN=128 selects the narrower tile for the tensor-core forms (tuning / comparison).
    static const int bn_env = [] { const char* v = getenv("TFP8B_W8A8_BN"); return v ? atoi(v) : 0; }();
    const bool wide = bn_env != 128;
    if (scale_mode == TFP8B_W8A8_ROWCOL)
        return wide ? launch_mx<MXM_ROWCOL, 192>(a_codes, w_codes, p, st) : launch_mx<MXM_ROWCOL, 128>(a_codes, w_codes, p, st);
    if (scale_kind == TFP8B_SCALE_UE8M0)
        return wide ? launch_mx<MXM_BLOCK_E8, 192>(a_codes, w_codes, p, st) : launch_mx<MXM_BLOCK_E8, 128>(a_codes, w_codes, p, st);
    return launch_mx<MXM_BLOCK_F32, 128>(a_codes, w_codes, p, st);      // accumulates a tile's columns in registers: 128 of them
}
