// Decode GEMV for 1 <= M <= 8 activation rows (kernel a).
//
//   y[m,n] = sum_g scale[n,g] * sum_{k in g} x[m,k] * dec(codes[n,k]) + bias[n]
//
// The weight stream is the whole cost (N*K bytes against M*(K+N) activation elements), so the
// kernel is built around keeping HBM busy from its first to its last microsecond:
//   * persistent CTAs, one per SM (two resident: this kernel's and its successor's), each walking
//     a list of 16-row weight tiles; K is cut into stages of 1024 codes that flow through one ring
//     of shared-memory stages which does not drain between tiles;
//   * a producer warp moves each stage with ONE 3-D tensor-map load (16 rows x 8 k-blocks of 128
//     bytes, 128-byte swizzle, evict-first in L2), completion counted in bytes on an mbarrier -- no
//     registers are held for data in flight. A K that is not a multiple of 128 takes the other
//     layout: 16 row pieces per stage by 1-D bulk copies into padded rows;
//   * the activations are copied into shared memory once per CTA when they fit (always for
//     M = 1), otherwise they travel with each stage through a tensor map of their own; two
//     further instantiations compute them in the kernel instead (residual + RMSNorm, SwiGLU);
//   * sixteen consumer warps each take a 64-code slice of a stage: 128-bit shared loads, two
//     codes per conversion instruction (see dec2_f16), products on the tensor cores with
//     mma.sync.m16n8k16 (16 weight rows x 8 activation rows, FP32 accumulate): at M = 8 the
//     FP32 FMA pipe could not keep up with HBM3e's byte rate, the MMA makes M irrelevant;
//   * x is consumed in its own type: f16 -> f16 MMA; bf16 -> bf16 MMA against weights decoded
//     to bf16 (every FP8 value is exact in both); f32 -> three bf16 terms (24 mantissa bits) and
//     three MMAs. Nothing is rounded before the FP32 accumulation;
//   * per-K-group scales multiply each group's partial sum in FP32 (exact for any scale value),
//     per-channel scales once at the end; the sixteen partial sums of a tile are handed to an
//     epilogue warp through one of two buffers and added in a fixed order, so results are
//     deterministic and the consumers never wait for the stores;
//   * programmatic dependent launch: the kernel releases its successor at once and only waits
//     for its predecessor before it touches activations or outputs, so in a chain of layers the
//     next layer's weights are already streaming while this one finishes. (The kernel before a
//     GEMV in its stream must therefore not write that GEMV's weights: see include/tfp8b.h.)
// All mbarrier waits are bounded; a wait that runs out sets a status bit and ends the CTA.
#include <stdlib.h>

#include "common.cuh"

namespace tfp8b {

constexpr int GV_ROWS = 16;                      // weight rows per tile (the MMA's M)
#ifndef TFP8B_GV_WARPS
#define TFP8B_GV_WARPS 16
#endif
constexpr int GV_WARPS = TFP8B_GV_WARPS;         // consumer warps
constexpr int GV_CONSUMERS = GV_WARPS * 32;
constexpr int GV_THREADS = GV_CONSUMERS + 64;    // + one producer warp + one epilogue warp
#ifndef TFP8B_GV_KS
#define TFP8B_GV_KS 1024
#endif
#ifndef TFP8B_GV_SMEM_KB
#define TFP8B_GV_SMEM_KB 104
#endif
constexpr int GV_KS = TFP8B_GV_KS;               // codes of K per stage
constexpr int GV_WK = GV_KS / GV_WARPS;          // codes of K per warp per stage
constexpr int GV_MAX_STAGES = 14;
constexpr int GV_RED = GV_WARPS * GV_ROWS * 8 * 4;            // one reduction buffer
constexpr int GV_HEADER = (384 + 2 * GV_RED + 1023) / 1024 * 1024;   // barriers + two reduction buffers, padded to 1 KB
constexpr int GV_SMEM_TARGET = TFP8B_GV_SMEM_KB * 1024;       // per CTA: two CTAs (this kernel + its successor) share an SM
constexpr int GV_SMEM_LARGE = 200 * 1024;        // ... unless the activations need the room (M > 1 with a long K)
constexpr int GV_XRES_SMALL = 40 * 1024;         // resident activations up to this size keep the small footprint
constexpr int GV_XRES_MAX = 96 * 1024;           // activations up to this size stay resident per CTA

struct GemvParams {
    const void* x;
    const uint8_t* w;
    const void* scale;
    const float* bias;
    void* y;
    int M, N, K, G, scale_kind, y_dt;
    int nstages, wpitch, xpitch, wstage_bytes, stage_bytes, x_resident, xres_bytes, ntiles, pdl;
    int trig;                 // when the kernel releases its dependents: 0 at its start, 1 once its last weight stage is requested
    // Activations computed by the kernel itself instead of copied (16-bit types, resident rows):
    //   xmode 1  x = RMSNorm(xa + xb) * xw: the residual update (xb may be null) and the norm of a
    //            decoder block; the CTA with index 0 also stores the updated residual to xout
    //   xmode 2  x = silu(xa[:, 0:K]) * xa[:, K:2K]: the gated activation of a fused gate/up output
    // Every CTA recomputes the few rows (they come from L2); what it saves is a kernel in the
    // dependent chain of a decode step.
    int xmode;
    const void* xa;
    const void* xb;
    const void* xw;
    void* xout;
    float xeps;
};

__device__ __forceinline__ void mma16816_f16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Two floats -> packed bf16x2 (low half = first), round to nearest even.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float bf16_lo(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }

// One MMA step: four codes of weight row g (word wa) and of row g+8 (word wb) against four
// activations of row m. The K positions inside an MMA are permuted the same way on both operands
// (lane tig owns 16 consecutive k), which leaves the dot product unchanged and lets every lane
// load whole 16-byte pieces.
//   f16 / bf16 x: xq[0] = {x0,x1}, xq[1] = {x2,x3} as stored.
//   f32 x       : xq[0..3] = x0..x3 as float bits, split into three bf16 terms.
template <typename XT, int FMT>
__device__ __forceinline__ void mma_step(float c[4], uint32_t wa, uint32_t wb, const uint32_t* xq) {
    constexpr bool BF = dtype_of<XT>::id != TFP8B_F16;
    uint32_t a0, a1, a2, a3;
    dec4<FMT, BF>(wa, a0, a2);
    dec4<FMT, BF>(wb, a1, a3);
    if (dtype_of<XT>::id == TFP8B_F16) {
        mma16816_f16(c, a0, a1, a2, a3, xq[0], xq[1]);
    } else if (dtype_of<XT>::id == TFP8B_BF16) {
        mma16816_bf16(c, a0, a1, a2, a3, xq[0], xq[1]);
    } else {
        float f0 = __uint_as_float(xq[0]), f1 = __uint_as_float(xq[1]);
        float f2 = __uint_as_float(xq[2]), f3 = __uint_as_float(xq[3]);
#pragma unroll
        for (int term = 0; term < 3; ++term) {
            uint32_t b0 = pack_bf16(f0, f1), b1 = pack_bf16(f2, f3);
            mma16816_bf16(c, a0, a1, a2, a3, b0, b1);
            f0 -= bf16_lo(b0); f1 -= bf16_hi(b0); f2 -= bf16_lo(b1); f3 -= bf16_hi(b1);
        }
    }
}

// The MMA steps of a block go to separate accumulators c[0..3], so that no mma.sync waits for the
// one before it.
//
// Shared-memory loads by 32-bit shared-window address: no generic-pointer arithmetic in the inner
// loop (the first version spent 3.5 instructions per code, most of them on addresses).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}

// A 64-code block of the stage: lane (g, tig) takes the 16 codes at k = kofs + 16*tig of tile rows
// R (address wa) and R+8 (address wb) and the matching 16 activations of row m, found as XCH
// 16-byte pieces at xb + xoff[i]. MASK (bulk-copy layout only): the block is only half inside K
// (K is a multiple of 32), lanes with tig >= 2 contribute zeros.
template <typename XT, int FMT, bool MASK>
__device__ __forceinline__ void block64(float (*c)[4], uint32_t wa_addr, uint32_t wb_addr, uint32_t xb, const int* xoff, bool live) {
    uint4 wa = lds128(wa_addr);
    uint4 wb = lds128(wb_addr);
    constexpr int XW = sizeof(XT) == 4 ? 16 : 8;           // 32-bit words of x per lane per block
    uint32_t xr[XW];
#pragma unroll
    for (int i = 0; i < XW / 4; ++i) {
        uint4 v = lds128(xb + xoff[i]);
        xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
    }
    if (MASK && !live) {
        wa = make_uint4(0, 0, 0, 0); wb = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < XW; ++i) xr[i] = 0u;
    }
    const uint32_t was[4] = {wa.x, wa.y, wa.z, wa.w}, wbs[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) mma_step<XT, FMT>(c[j], was[j], wbs[j], &xr[j * (XW / 4)]);
}

// A 32-code block (32-wide scale groups): lane (g, tig) takes 8 codes at k = kofs + 8*tig.
template <typename XT, int FMT>
__device__ __forceinline__ void block32(float (*c)[4], uint32_t wa_addr, uint32_t wb_addr, uint32_t xb, const int* xoff) {
    uint2 wa = lds64(wa_addr);
    uint2 wb = lds64(wb_addr);
    constexpr int XW = sizeof(XT) == 4 ? 8 : 4;
    uint32_t xr[XW];
#pragma unroll
    for (int i = 0; i < XW / 4; ++i) {
        uint4 v = lds128(xb + xoff[i]);
        xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
    }
    mma_step<XT, FMT>(c[0], wa.x, wb.x, &xr[0]);
    mma_step<XT, FMT>(c[1], wa.y, wb.y, &xr[XW / 2]);
}

// Which weight row of the 16-row tile sits in MMA row g (0..7; MMA row g+8 holds that row + 8).
// 16-bit pair helpers for the computed-activation modes
__device__ __forceinline__ float2 gv_unpack(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 gv_unpack(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ float2 gv_unpack(float2 v) { return v; }
template <typename P> __device__ __forceinline__ P gv_pack(float a, float b);
template <> __device__ __forceinline__ __half2 gv_pack<__half2>(float a, float b) { return __floats2half2_rn(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 gv_pack<__nv_bfloat162>(float a, float b) { return __floats2bfloat162_rn(a, b); }
template <> __device__ __forceinline__ float2 gv_pack<float2>(float a, float b) { return make_float2(a, b); }
template <typename XT> struct gv_pair { using type = float2; };
template <> struct gv_pair<__half> { using type = __half2; };
template <> struct gv_pair<__nv_bfloat16> { using type = __nv_bfloat162; };

// The consumer warps (GV_WARPS * 32 threads) fill the resident activation rows themselves. `scratch`
// is the (still unused) reduction area of the header. Named barrier 2 is theirs alone.
template <typename XT>
__device__ __forceinline__ void compute_activations(const GemvParams& p, uint8_t* xres, float* scratch, int warp, int lane) {
    using P = typename gv_pair<XT>::type;
    constexpr int NT = GV_WARPS * 32;
    const int tid = warp * 32 + lane, nvec = p.K / 8;
    if (sizeof(XT) != 2) return;                                   // 16-bit activations only (checked on the host)
    if (p.xmode == 2) {
        const XT* gu = reinterpret_cast<const XT*>(p.xa);
        for (int m = 0; m < p.M; ++m) {
            const XT* row = gu + static_cast<size_t>(m) * 2 * p.K;
            for (int v = tid; v < nvec; v += NT) {
                const uint4 g = *reinterpret_cast<const uint4*>(row + v * 8);
                const uint4 u = *reinterpret_cast<const uint4*>(row + p.K + v * 8);
                const P* gp = reinterpret_cast<const P*>(&g);
                const P* up = reinterpret_cast<const P*>(&u);
                uint4 o;
                P* op = reinterpret_cast<P*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 a = gv_unpack(gp[i]), b = gv_unpack(up[i]);
                    op[i] = gv_pack<P>(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
                }
                *reinterpret_cast<uint4*>(xres + m * p.xpitch + v * 16) = o;
            }
        }
        named_barrier_sync(2, NT);
        return;
    }
    // xmode 1: residual (+ delta), rounded to the activation type, kept in shared memory; sum of squares
    const XT* ra = reinterpret_cast<const XT*>(p.xa);
    const XT* rb = reinterpret_cast<const XT*>(p.xb);
    XT* ro = reinterpret_cast<XT*>(p.xout);
    for (int m = 0; m < p.M; ++m) {
        float ss = 0.f;
        for (int v = tid; v < nvec; v += NT) {
            uint4 a = *reinterpret_cast<const uint4*>(ra + static_cast<size_t>(m) * p.K + v * 8);
            P* ap = reinterpret_cast<P*>(&a);
            if (rb) {
                const uint4 d = *reinterpret_cast<const uint4*>(rb + static_cast<size_t>(m) * p.K + v * 8);
                const P* dp = reinterpret_cast<const P*>(&d);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = gv_unpack(ap[i]), g = gv_unpack(dp[i]);
                    ap[i] = gv_pack<P>(f.x + g.x, f.y + g.y);
                }
            }
            if (ro && blockIdx.x == 0) *reinterpret_cast<uint4*>(ro + static_cast<size_t>(m) * p.K + v * 8) = a;
            *reinterpret_cast<uint4*>(xres + m * p.xpitch + v * 16) = a;
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = gv_unpack(ap[i]); ss += f.x * f.x + f.y * f.y; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) scratch[m * GV_WARPS + warp] = ss;
    }
    named_barrier_sync(2, NT);
    const XT* wv = reinterpret_cast<const XT*>(p.xw);
    for (int m = 0; m < p.M; ++m) {
        float ss = 0.f;
#pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) ss += scratch[m * GV_WARPS + w];
        const float rstd = rsqrtf(ss / static_cast<float>(p.K) + p.xeps);
        for (int v = tid; v < nvec; v += NT) {
            uint4 a = *reinterpret_cast<const uint4*>(xres + m * p.xpitch + v * 16);
            const uint4 wq = *reinterpret_cast<const uint4*>(wv + v * 8);
            P* ap = reinterpret_cast<P*>(&a);
            const P* wp = reinterpret_cast<const P*>(&wq);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = gv_unpack(ap[i]), g = gv_unpack(wp[i]);
                ap[i] = gv_pack<P>(f.x * rstd * g.x, f.y * rstd * g.y);
            }
            *reinterpret_cast<uint4*>(xres + m * p.xpitch + v * 16) = a;
        }
    }
    named_barrier_sync(2, NT);
}

// With the tensor-map layout the rows of a tile are 128 bytes apart and the 16-byte pieces of a
// row are XOR-swizzled with (row & 7): the permutation puts rows that differ in the right bit
// into the lanes that load together, which makes the loads bank-conflict free (128-bit loads go
// by quarter warps = MMA rows {2q, 2q+1}; 64-bit loads by half warps = MMA rows {4h..4h+3}).
// Any permutation is legal: it only decides which output row a lane's accumulator belongs to.
template <int SMODE, bool TMA>
__device__ __forceinline__ int tile_row_of(int g) {
    if (!TMA) return g;
    return SMODE == 2 ? 2 * (g & 3) + (g >> 2) : (g >> 1) + 4 * (g & 1);
}

// Shared-memory map:  [0,256) mbarriers: full[0..13], empty[14..27], xfull[28], red_full[29..30], red_empty[31..32]
//                     [384, 384 + 2*GV_RED) two reduction buffers [warp][row][m]
//                     (1024-byte aligned) resident activations, then the ring of stages.
// Two data layouts:
//   TMA   (K % 128 == 0) one 3-D tensor-map load per stage brings 16 rows x 1024 codes as
//         [8 k-blocks][16 rows][128 B] with the 128-byte swizzle; activations that travel with
//         the stage likewise as [k-blocks][M rows][128 B]. One instruction per 16 KB: issuing
//         one bulk copy per 1 KB row piece, as the other layout does, capped a CTA at ~20 GB/s.
//   bulk  (any K % 32 == 0) 16 row pieces of up to 1 KB by cp.async.bulk, row pitch padded for
//         conflict-free loads; used for the K that the tensor map cannot describe.
//
// SMODE 0: one scale per output channel (applied once, at the end)
//       1: K-groups that are multiples of 64 (applied per 64-code block)
//       2: K-groups that are multiples of 32 only (32-code blocks)
// XF: the activations are computed by the kernel (GemvParams::xmode) instead of copied. A template
// parameter, not a run-time branch: the plain kernel stays exactly the code it was (the branch
// alone cost it 1 % of its bandwidth).
template <typename XT, int FMT, int SMODE, bool TMA, bool XF>
__global__ void __launch_bounds__(GV_THREADS, 2)
gemv_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemvParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    float* red = reinterpret_cast<float*>(smem + 384);
    uint8_t* xres = smem + GV_HEADER;
    uint8_t* stages = xres + p.xres_bytes;
    const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[GV_MAX_STAGES]);
    const uint32_t bar_x = smem_u32(&bars[2 * GV_MAX_STAGES]);
    const uint32_t bar_red_full = smem_u32(&bars[2 * GV_MAX_STAGES + 1]);     // [2]: partial sums of a tile written
    const uint32_t bar_red_empty = smem_u32(&bars[2 * GV_MAX_STAGES + 3]);    // [2]: ... and read by the epilogue warp
    constexpr int SZ = static_cast<int>(sizeof(XT));
    constexpr int EPB = 128 / SZ;                    // activations per 128-byte k-block (TMA layout)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = p.nstages;
    const int nchunks = (p.K + GV_KS - 1) / GV_KS;
    const int my_tiles = (p.ntiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
    const int total = my_tiles * nchunks;            // stages this CTA moves in all

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, GV_WARPS);
        }
        mbar_init(bar_x, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_red_full + 8 * b, GV_WARPS);
            mbar_init(bar_red_empty + 8 * b, 1);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
        if (TMA) { tma_prefetch_desc(&tm_w); tma_prefetch_desc(&tm_x); }
    }
    __syncthreads();
    if (p.pdl && p.trig == 0) pdl_launch_dependents();

    if (warp == GV_WARPS) {
        // ---------------------------------------------------------------- producer warp
        const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
        const int xm = lane - 16;
        const uint8_t* xrow = reinterpret_cast<const uint8_t*>(p.x) + static_cast<size_t>(max(xm, 0)) * p.K * SZ;
        // bytes of activations that travel with a stage, per code of K (bulk) or per stage (TMA)
        const uint32_t x_per_k = p.x_resident ? 0u : static_cast<uint32_t>(p.M * SZ);

        // (t, c, slot) name the stage being issued: tile of this CTA, chunk of K, ring slot
        auto issue_w = [&](int t, int c, int slot) {
            const int n0 = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * GV_ROWS;
            const int k0 = c * GV_KS, klen = min(GV_KS, p.K - k0);
            uint8_t* wst = stages + static_cast<size_t>(slot) * p.stage_bytes;
            if (TMA) {
                if (lane == 0) {
                    mbar_expect_tx(bar_full + 8 * slot, static_cast<uint32_t>(GV_KS) * (GV_ROWS + x_per_k));
                    tma_load_3d(smem_u32(wst), &tm_w, 0, n0, k0 >> 7, bar_full + 8 * slot, pol_w);
                }
            } else {
                if (lane == 0) mbar_expect_tx(bar_full + 8 * slot, static_cast<uint32_t>(klen) * (GV_ROWS + x_per_k));
                __syncwarp();
                if (lane < GV_ROWS) {
                    const int row = min(n0 + lane, p.N - 1);             // N tail: re-read the last row
                    bulk_g2s(smem_u32(wst + lane * p.wpitch), p.w + static_cast<size_t>(row) * p.K + k0, klen,
                             bar_full + 8 * slot, pol_w);
                }
            }
        };
        auto issue_x = [&](int c, int slot) {                            // activations that travel with the stage
            const int k0 = c * GV_KS, klen = min(GV_KS, p.K - k0);
            uint8_t* xst = stages + static_cast<size_t>(slot) * p.stage_bytes + p.wstage_bytes;
            if (TMA) {
                if (lane == 0) tma_load_3d(smem_u32(xst), &tm_x, 0, 0, k0 / EPB, bar_full + 8 * slot, pol_x);
            } else if (xm >= 0 && xm < p.M) {
                bulk_g2s(smem_u32(xst + xm * p.xpitch), xrow + static_cast<size_t>(k0) * SZ, klen * SZ, bar_full + 8 * slot, pol_x);
            }
        };

        const int pre = min(S, total);
        int t = 0, c = 0;
        for (int i = 0; i < pre; ++i) {                  // weights first: they never depend on the predecessor
            issue_w(t, c, i);
            if (++c == nchunks) { c = 0; ++t; }
        }
        if (p.pdl == 1) pdl_wait();                      // activations may be the predecessor's output
        if (p.x_resident && !XF) {
            // resident activations: plain rows (pitch xpitch), loaded once per CTA by bulk copies
            if (lane == 0) mbar_expect_tx(bar_x, static_cast<uint32_t>(p.M * p.K * SZ));
            __syncwarp();
            if (xm >= 0 && xm < p.M) {
                // one row can exceed what a single bulk copy should carry: cut it at 16 KB
                for (int off = 0; off < p.K * SZ; off += 16384)
                    bulk_g2s(smem_u32(xres + xm * p.xpitch + off), xrow + off, min(16384, p.K * SZ - off), bar_x, pol_x);
            }
        } else if (!p.x_resident) {
            int cx = 0;
            for (int i = 0; i < pre; ++i) {
                issue_x(cx, i);
                if (++cx == nchunks) cx = 0;
            }
        }
        int slot = 0;
        uint32_t phase = 0;                              // parity of the slot's previous use
        for (int i = pre; i < total; ++i) {
            if (!mbar_wait(bar_empty + 8 * slot, phase, STATUS_GEMV_WAIT)) break;
            issue_w(t, c, slot);
            if (!p.x_resident) issue_x(c, slot);
            if (++c == nchunks) { c = 0; ++t; }
            if (++slot == S) { slot = 0; phase ^= 1u; }
        }
        // every byte this CTA will ask of HBM has been requested: from here on a successor's
        // weight prefetch competes with nothing of this kernel
        if (p.pdl && p.trig == 1) pdl_launch_dependents();
    } else if (warp < GV_WARPS) {
        // ---------------------------------------------------------------- consumer warps
        const int g = lane >> 2, tig = lane & 3;
        const int R = tile_row_of<SMODE, TMA>(g);        // tile rows R and R + 8 live in this lane's MMA rows
        const int mrow = min(g, p.M - 1);
        const int ng = p.K / p.G;
        constexpr int BLK = SMODE == 2 ? 32 : 64;
        constexpr int NB = GV_WK / BLK;
        constexpr int XCH = BLK * SZ / 64;               // 16-byte pieces of x per lane per block
        const int kw = warp * GV_WK;
        // Lane-constant shared-memory offsets of this lane's operands inside a stage (weights) and
        // relative to the activations of the stage's first code (x), one set per block.
        int woff[NB], xoff[NB][XCH];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int kk = kw + b * BLK + tig * (BLK / 4);           // this lane's first code within the stage
            if (TMA) woff[b] = (kk >> 7) * 2048 + R * 128 + ((((kk >> 4) & 7) ^ R) << 4) + (kk & 8);
            else woff[b] = R * p.wpitch + kk;
            if (TMA && !p.x_resident) {
                const int xo = ((kk / EPB) * p.M + mrow) * 128, ph = (xo >> 7) & 7, c0 = ((kk % EPB) * SZ) >> 4;
#pragma unroll
                for (int i = 0; i < XCH; ++i) xoff[b][i] = xo + (((c0 + i) ^ ph) << 4);
            } else {
#pragma unroll
                for (int i = 0; i < XCH; ++i) xoff[b][i] = mrow * p.xpitch + kk * SZ + 16 * i;
            }
        }
        const uint32_t stages_u32 = smem_u32(stages), xres_u32 = smem_u32(xres);
        bool ok = true;
        if (XF) {
            if (p.pdl) pdl_wait();                       // the inputs are the predecessor's output
            compute_activations<XT>(p, xres, red, warp, lane);
        } else if (p.x_resident) {
            ok = mbar_wait(bar_x, 0, STATUS_GEMV_WAIT);
        }
        int slot = 0;
        uint32_t phase = 0;                              // ring position: no divisions in the loop
        // A wait that runs out clears `ok`; the warp then stops waiting and computing but keeps
        // walking the loop, so it still meets the others at every barrier and the CTA ends.
        for (int t = 0; t < my_tiles; ++t) {
            const int n0 = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * GV_ROWS;
            const size_t srow_a = static_cast<size_t>(min(n0 + R, p.N - 1)) * ng;
            const size_t srow_b = static_cast<size_t>(min(n0 + R + 8, p.N - 1)) * ng;
            // SMODE 0 accumulates straight into eight independent MMA accumulators (block parity x
            // step); the grouped modes sum each block's four partials and apply the group scale.
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            float cc[8][4];
#pragma unroll
            for (int a = 0; a < 8; ++a) cc[a][0] = cc[a][1] = cc[a][2] = cc[a][3] = 0.f;
            for (int c = 0; c < nchunks; ++c) {
                const int cur = slot;
                const uint32_t par = phase;
                if (++slot == S) { slot = 0; phase ^= 1u; }
                const int k0 = c * GV_KS, klen = min(GV_KS, p.K - k0);
                float sa[NB], sb[NB];
                if (SMODE != 0) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        sa[b] = sb[b] = 0.f;
                        if (kw + b * BLK < klen) {
                            const int gi = (k0 + kw + b * BLK) / p.G;
                            sa[b] = load_scale(p.scale, srow_a + gi, p.scale_kind);
                            sb[b] = load_scale(p.scale, srow_b + gi, p.scale_kind);
                        }
                    }
                }
                if (ok) ok = mbar_wait(bar_full + 8 * cur, par, STATUS_GEMV_WAIT);
                if (!ok) continue;
                const uint32_t wst = stages_u32 + static_cast<uint32_t>(cur * p.stage_bytes);
                // activations: the resident rows at this stage's first code, or the stage's own piece
                const uint32_t xb = p.x_resident ? xres_u32 + static_cast<uint32_t>(k0 * SZ) : wst + static_cast<uint32_t>(p.wstage_bytes);
                const uint32_t wrow8 = TMA ? 1024u : static_cast<uint32_t>(8 * p.wpitch);   // tile row R + 8
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const int kofs = kw + b * BLK;
                    if (kofs < klen) {
                        const uint32_t wa = wst + woff[b], wb = wa + wrow8;
                        const bool live = kofs + tig * (BLK / 4) < klen;
                        if (SMODE == 0) {
                            float (*cb)[4] = &cc[(b & 1) * 4];
                            if (TMA || kofs + 64 <= klen) block64<XT, FMT, false>(cb, wa, wb, xb, xoff[b], true);
                            else block64<XT, FMT, true>(cb, wa, wb, xb, xoff[b], live);
                        } else {
                            float tt[4][4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) tt[q][0] = tt[q][1] = tt[q][2] = tt[q][3] = 0.f;
                            if (SMODE == 2) block32<XT, FMT>(tt, wa, wb, xb, xoff[b]);
                            else if (TMA || kofs + 64 <= klen) block64<XT, FMT, false>(tt, wa, wb, xb, xoff[b], true);
                            else block64<XT, FMT, true>(tt, wa, wb, xb, xoff[b], live);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float t4 = (tt[0][e] + tt[1][e]) + (tt[2][e] + tt[3][e]);
                                acc[e] = fmaf(t4, e < 2 ? sa[b] : sb[b], acc[e]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * cur);
            }
            if (SMODE == 0) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    acc[e] = ((cc[0][e] + cc[1][e]) + (cc[2][e] + cc[3][e])) + ((cc[4][e] + cc[5][e]) + (cc[6][e] + cc[7][e]));
            }
            // Hand the eight K-slices' partial sums to the epilogue warp through one of two
            // buffers, so that the consumers go straight on with the next tile: the reduction, the
            // scale / bias loads and the stores are off their critical path.
            if (ok && t >= 2) ok = mbar_wait(bar_red_empty + 8 * (t & 1), ((t >> 1) - 1) & 1, STATUS_GEMV_WAIT);
            float* r = red + (t & 1) * (GV_RED / 4) + warp * (GV_ROWS * 8);
            r[R * 8 + 2 * tig] = acc[0];
            r[R * 8 + 2 * tig + 1] = acc[1];
            r[(R + 8) * 8 + 2 * tig] = acc[2];
            r[(R + 8) * 8 + 2 * tig + 1] = acc[3];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_red_full + 8 * (t & 1));
        }
    } else {
        // ---------------------------------------------------------------- epilogue warp
        // lane -> four outputs (row, m) of the 16 x 8 tile; the eight partial sums are added in a
        // fixed order, so the result does not depend on timing.
        bool ok = true;
        if (p.pdl == 1) pdl_wait();                      // before the first store to y
        for (int t = 0; t < my_tiles; ++t) {
            const int n0 = (static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x)) * GV_ROWS;
            const int row = lane & 15, n = n0 + row;
            const bool live = n < p.N;
            const float bv = (live && p.bias) ? p.bias[n] : 0.f;
            const float sv = (live && SMODE == 0) ? load_scale(p.scale, n, p.scale_kind) : 1.f;
            if (ok) ok = mbar_wait(bar_red_full + 8 * (t & 1), (t >> 1) & 1, STATUS_GEMV_WAIT);
            if (ok) {
                const float* rb = red + (t & 1) * (GV_RED / 4);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int m = (lane >> 4) + 2 * j;
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < GV_WARPS; ++w) v += rb[w * (GV_ROWS * 8) + row * 8 + m];
                    v = SMODE == 0 ? fmaf(v, sv, bv) : v + bv;
                    if (live && m < p.M) store_dt(p.y, static_cast<size_t>(m) * p.N + n, v, p.y_dt);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_red_empty + 8 * (t & 1));
        }
        if (p.pdl == 2) pdl_wait();                      // independent I/O: only completion is ordered
    }
}

// SM count of the current device, asked once per device (the query sits on the launch path of
// kernels that take a few microseconds).
static int sm_count_of_current_device() {
    static int cached[64] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

template <typename XT, int FMT, int SMODE, bool TMA, bool XF>
static int launch_gemv(const CUtensorMap& tw, const CUtensorMap& tx, const GemvParams& p, size_t smem, cudaStream_t st) {
    // The opt-in to more than 48 KB of dynamic shared memory is per device and per kernel.
    static unsigned long long configured = 0ull;        // bit d set: done on device d
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev >= 64 || !((configured >> dev) & 1ull)) {
        e = cudaFuncSetAttribute(gemv_kernel<XT, FMT, SMODE, TMA, XF>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemv)");
        if (dev < 64) __atomic_fetch_or(&configured, 1ull << dev, __ATOMIC_RELAXED);
    }
    const int sms = sm_count_of_current_device();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p.ntiles < sms ? p.ntiles : sms));
    cfg.blockDim = dim3(GV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, gemv_kernel<XT, FMT, SMODE, TMA, XF>, tw, tx, p);
    if (e != cudaSuccess) return cuda_fail(e, "tfp8b_gemv launch");
    return TFP8B_OK;
}

template <typename XT>
static int dispatch_gemv(const CUtensorMap& tw, const CUtensorMap& tx, const GemvParams& p, int fmt, int smode, bool tma,
                         size_t smem, cudaStream_t st) {
    if (p.xmode != 0) {          // computed activations: 16-bit types on the tensor-map layout only (checked by the caller)
        if (sizeof(XT) == 2) {
#define GV_CASE(F, S) if (fmt == F && smode == S) return launch_gemv<XT, F, S, true, (sizeof(XT) == 2)>(tw, tx, p, smem, st)
            GV_CASE(TFP8B_E4M3FN, 0); GV_CASE(TFP8B_E4M3FN, 1); GV_CASE(TFP8B_E4M3FN, 2);
            GV_CASE(TFP8B_E5M2, 0);   GV_CASE(TFP8B_E5M2, 1);   GV_CASE(TFP8B_E5M2, 2);
#undef GV_CASE
        }
        set_error("tfp8b_gemv: computed activations need f16 / bf16");
        return TFP8B_ERR_UNSUPPORTED;
    }
#define GV_CASE(F, S)                                                                   \
    if (fmt == F && smode == S)                                                         \
        return tma ? launch_gemv<XT, F, S, true, false>(tw, tx, p, smem, st) : launch_gemv<XT, F, S, false, false>(tw, tx, p, smem, st)
    GV_CASE(TFP8B_E4M3FN, 0); GV_CASE(TFP8B_E4M3FN, 1); GV_CASE(TFP8B_E4M3FN, 2);
    GV_CASE(TFP8B_E5M2, 0);   GV_CASE(TFP8B_E5M2, 1);   GV_CASE(TFP8B_E5M2, 2);
#undef GV_CASE
    set_error("tfp8b_gemv: bad fmt %d", fmt);
    return TFP8B_ERR_INVALID;
}

int gemv_status(unsigned int* out, cudaStream_t st) {
    unsigned int* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&word), g_status);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(gemv status)");
    return read_and_clear_status(word, out, st);
}

}  // namespace tfp8b

using namespace tfp8b;

extern "C" int tfp8b_gemv(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
                          const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                          tfp8b_stream_t stream) {
    return tfp8b_gemv_ex(x, x_dtype, codes, scale, scale_kind, bias, y, y_dtype, M, N, K, G, fmt, 0u, stream);
}

static int gemv_impl(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind, const float* bias,
                     void* y, int y_dtype, int M, int N, int K, int G, int fmt, unsigned int flags, int xmode, const void* xa,
                     const void* xb, const void* xw, void* xout, float xeps, tfp8b_stream_t stream);

extern "C" int tfp8b_gemv_ex(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
                             const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                             unsigned int flags, tfp8b_stream_t stream) {
    return gemv_impl(x, x_dtype, codes, scale, scale_kind, bias, y, y_dtype, M, N, K, G, fmt, flags, 0, nullptr, nullptr, nullptr,
                     nullptr, 0.f, stream);
}

extern "C" int tfp8b_gemv_normed(void* residual_out, const void* residual, const void* delta, const void* norm_weight, float eps,
                                 int x_dtype, const uint8_t* codes, const void* scale, int scale_kind, const float* bias, void* y,
                                 int y_dtype, int M, int N, int K, int G, int fmt, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(x_dtype == TFP8B_F16 || x_dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_gemv_normed: f16 / bf16 activations only");
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(residual && norm_weight, TFP8B_ERR_INVALID, "tfp8b_gemv_normed: null pointer");
    TFP8B_REQUIRE(residual_out != residual || !delta, TFP8B_ERR_INVALID,
                  "tfp8b_gemv_normed: the updated residual needs a buffer of its own (every CTA reads the old one)");
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(norm_weight) |
                    reinterpret_cast<uintptr_t>(residual_out)) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_gemv_normed: buffers must be 16-byte aligned");
    return gemv_impl(residual, x_dtype, codes, scale, scale_kind, bias, y, y_dtype, M, N, K, G, fmt, 0u, 1, residual, delta, norm_weight,
                     residual_out, eps, stream);
}

extern "C" int tfp8b_gemv_gated(const void* gate_up, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind,
                                const float* bias, void* y, int y_dtype, int M, int N, int K, int G, int fmt,
                                tfp8b_stream_t stream) {
    TFP8B_REQUIRE(x_dtype == TFP8B_F16 || x_dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_gemv_gated: f16 / bf16 activations only");
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(gate_up && (reinterpret_cast<uintptr_t>(gate_up) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_gemv_gated: gate_up null or unaligned");
    return gemv_impl(gate_up, x_dtype, codes, scale, scale_kind, bias, y, y_dtype, M, N, K, G, fmt, 0u, 2, gate_up, nullptr, nullptr,
                     nullptr, 0.f, stream);
}

// Everything of a launch that does not depend on the addresses of x and y: shape checks, the
// shared-memory plan, the kernel variant, the tensor map of the weight stream.
struct GemvSetup {
    GemvParams p;
    CUtensorMap tw;
    size_t smem;
    int fmt, smode, x_dtype;
    bool tma;
};

static int gemv_weight_map(CUtensorMap* tw, const uint8_t* codes, int N, int K) {
    // weights: [k-block][row][128 B]; dim 1 (rows) strides by K, dim 2 (k-blocks) by 128 bytes
    const cuuint64_t wd[3] = {128, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K / 128)};
    const cuuint64_t ws[2] = {static_cast<cuuint64_t>(K), 128};
    const cuuint32_t wb[3] = {128, GV_ROWS, GV_KS / 128};
    return encode_tensor_map(tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, codes, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
}

static int gemv_x_map(CUtensorMap* tx, const void* x, int x_dtype, int M, int K) {
    const int xsz = dtype_size(x_dtype), epb = 128 / xsz;      // activations per 128-byte k-block
    const cuuint64_t xd[3] = {static_cast<cuuint64_t>(epb), static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(K / epb)};
    const cuuint64_t xs[2] = {static_cast<cuuint64_t>(K) * xsz, 128};
    const cuuint32_t xb[3] = {static_cast<cuuint32_t>(epb), static_cast<cuuint32_t>(M), static_cast<cuuint32_t>(GV_KS / epb)};
    const CUtensorMapDataType xt = x_dtype == TFP8B_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : x_dtype == TFP8B_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    return encode_tensor_map(tx, xt, 3, x, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B);
}

static int gemv_setup(GemvSetup& g, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind, const float* bias,
                      int y_dtype, int M, int N, int K, int G, int fmt, int xmode, bool with_weight_map) {
    TFP8B_REQUIRE(M >= 0 && N >= 0 && K > 0 && G > 0, TFP8B_ERR_INVALID, "tfp8b_gemv: bad size M=%d N=%d K=%d G=%d", M, N, K, G);
    TFP8B_REQUIRE(x_dtype >= 0 && x_dtype <= 2 && y_dtype >= 0 && y_dtype <= 2, TFP8B_ERR_INVALID, "tfp8b_gemv: bad dtype");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_gemv: bad fmt %d", fmt);
    TFP8B_REQUIRE(scale_kind == TFP8B_SCALE_F32 || scale_kind == TFP8B_SCALE_UE8M0, TFP8B_ERR_INVALID,
                  "tfp8b_gemv: bad scale_kind %d", scale_kind);
    TFP8B_REQUIRE(M <= 8, TFP8B_ERR_UNSUPPORTED, "tfp8b_gemv: M=%d > 8, use tfp8b_gemm", M);
    g.p = GemvParams{};
    g.fmt = fmt; g.x_dtype = x_dtype; g.smem = 0; g.smode = 0; g.tma = false;
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(codes && scale, TFP8B_ERR_INVALID, "tfp8b_gemv: null pointer");
    TFP8B_REQUIRE(K % 32 == 0 && G % 32 == 0 && K % G == 0, TFP8B_ERR_UNSUPPORTED,
                  "tfp8b_gemv: need K %% 32 == 0, G %% 32 == 0, K %% G == 0 (K=%d G=%d)", K, G);
    TFP8B_REQUIRE((reinterpret_cast<uintptr_t>(codes) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_gemv: codes must be 16-byte aligned");
    const int smode = G == K ? 0 : (G % 64 == 0 ? 1 : 2);
    const int xsz = dtype_size(x_dtype);
    GemvParams& p = g.p;
    p.w = codes; p.scale = scale; p.bias = bias;
    p.M = M; p.N = N; p.K = K; p.G = G; p.scale_kind = scale_kind; p.y_dt = y_dtype;
    p.ntiles = (N + GV_ROWS - 1) / GV_ROWS;
    p.xmode = xmode;
    // TFP8B_GEMV_BULK=1 forces the bulk-copy layout.
    static const int force_bulk = [] { const char* v = getenv("TFP8B_GEMV_BULK"); return v && v[0] == '1'; }();
    // The tensor map describes K in whole 128-byte k-blocks: a K that is not a multiple of 128
    // would make its last k-block read past the row (and, on the last row, past the buffer).
    const bool tma = K % 128 == 0 && !force_bulk;
    const int nchunks = (K + GV_KS - 1) / GV_KS;
    const int xpad = smode == 2 ? 64 : 16;
    // Tuning knobs: TFP8B_GEMV_XRES_MAX=<bytes> lowers the size up to which activations stay resident
    // (larger ones then travel with the stages); TFP8B_GEMV_STREAM_SMALL=1 gives that streaming
    // form the small footprint (two CTAs per SM) instead of the large one.
    static const int xres_max = [] { const char* v = getenv("TFP8B_GEMV_XRES_MAX"); const int n = v ? atoi(v) : 0; return n > 0 && n < GV_XRES_MAX ? n : GV_XRES_MAX; }();
    static const int stream_small = [] { const char* v = getenv("TFP8B_GEMV_STREAM_SMALL"); return v && v[0] == '1'; }();
    if (tma) {
        p.wstage_bytes = GV_ROWS * GV_KS;
        p.x_resident = (M * (K * xsz + xpad) <= xres_max) ? 1 : 0;
        p.xpitch = K * xsz + xpad;                                      // resident rows only
        p.xres_bytes = p.x_resident ? ((M * p.xpitch + 1023) & ~1023) : 0;
        const int xstage = p.x_resident ? 0 : M * GV_KS * xsz;          // a multiple of 1024
        p.stage_bytes = p.wstage_bytes + xstage;
        if (with_weight_map) {
            const int rc = gemv_weight_map(&g.tw, codes, N, K);
            if (rc != TFP8B_OK) return rc;
        }
    } else {
        // Row pitches that keep the 128-bit (64-code blocks) or 64-bit (32-code blocks) shared
        // loads of a quarter / half warp on distinct banks.
        p.wpitch = GV_KS + (smode == 2 ? 32 : 64);
        p.wstage_bytes = GV_ROWS * p.wpitch;
        p.x_resident = (M * (K * xsz + xpad) <= GV_XRES_MAX) ? 1 : 0;
        p.xpitch = (p.x_resident ? K : GV_KS) * xsz + xpad;
        p.xres_bytes = p.x_resident ? ((M * p.xpitch + 1023) & ~1023) : 0;
        p.stage_bytes = (p.wstage_bytes + (p.x_resident ? 0 : M * p.xpitch) + 127) & ~127;
        if (with_weight_map) g.tw = CUtensorMap{};
    }
    TFP8B_REQUIRE(xmode == 0 || (p.x_resident && tma), TFP8B_ERR_UNSUPPORTED,
                  "tfp8b_gemv: computed activations need K %% 128 == 0 and M * K small enough to stay resident (M=%d K=%d)", M, K);
    const int target = ((p.x_resident && p.xres_bytes <= GV_XRES_SMALL) || (!p.x_resident && tma && stream_small)) ? GV_SMEM_TARGET : GV_SMEM_LARGE;
    int S = (target - 1024 - GV_HEADER - p.xres_bytes) / p.stage_bytes;
    S = S < 2 ? 2 : (S > GV_MAX_STAGES ? GV_MAX_STAGES : S);
    const int sms = sm_count_of_current_device();
    const int max_items = ((p.ntiles + sms - 1) / sms) * nchunks;     // stages the busiest CTA moves
    if (S > max_items) S = max_items;
    p.nstages = S;
    g.smem = 1024 + GV_HEADER + p.xres_bytes + static_cast<size_t>(S) * p.stage_bytes;
    g.smode = smode; g.tma = tma;
    return TFP8B_OK;
}

// pdl: 0 = plain launch; 1 = early launch, wait for the predecessor before touching x / y;
//      2 = early launch, caller vouches that x / y are independent of the predecessor: the wait
//          moves to the very end (so that this grid never completes before its predecessor and
//          later work in the stream still sees both finished).
// TFP8B_NO_PDL=1 in the environment turns programmatic dependent launch off everywhere
// (profilers serialise kernels anyway).
static int pdl_mode_of(unsigned int flags) {
    static const int no_pdl = [] { const char* v = getenv("TFP8B_NO_PDL"); return v && v[0] == '1'; }();
    if (no_pdl || (flags & TFP8B_GEMV_NO_PDL)) return 0;
    return (flags & TFP8B_GEMV_INDEPENDENT_IO) ? 2 : 1;
}

static int gemv_run(const GemvSetup& g, const void* x, void* y, unsigned int flags, const void* xa, const void* xb,
                    const void* xw, void* xout, float xeps, tfp8b_stream_t stream) {
    if (g.p.M == 0 || g.p.N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x && y, TFP8B_ERR_INVALID, "tfp8b_gemv: null pointer");
    TFP8B_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_gemv: x must be 16-byte aligned");
    GemvParams p = g.p;
    p.x = x; p.y = y; p.xa = xa; p.xb = xb; p.xw = xw; p.xout = xout; p.xeps = xeps;
    p.pdl = pdl_mode_of(flags);
    // TFP8B_GEMV_TRIGGER=1: release the dependents once the last weight stage is requested instead of
    // at the kernel's start (tuning; measured inside a decode step: no gain at batch 1 and 8, 7 % slower at 4)
    static const int trig = [] { const char* v = getenv("TFP8B_GEMV_TRIGGER"); return (v && v[0] == '1') ? 1 : 0; }();
    p.trig = trig;
    CUtensorMap tx = {};
    if (g.tma && !p.x_resident) {                 // activations that travel with the stages: their own tensor map
        const int rc = gemv_x_map(&tx, x, g.x_dtype, p.M, p.K);
        if (rc != TFP8B_OK) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g.x_dtype == TFP8B_F16) return dispatch_gemv<__half>(g.tw, tx, p, g.fmt, g.smode, g.tma, g.smem, st);
    if (g.x_dtype == TFP8B_BF16) return dispatch_gemv<__nv_bfloat16>(g.tw, tx, p, g.fmt, g.smode, g.tma, g.smem, st);
    return dispatch_gemv<float>(g.tw, tx, p, g.fmt, g.smode, g.tma, g.smem, st);
}

static int gemv_impl(const void* x, int x_dtype, const uint8_t* codes, const void* scale, int scale_kind, const float* bias,
                     void* y, int y_dtype, int M, int N, int K, int G, int fmt, unsigned int flags, int xmode, const void* xa,
                     const void* xb, const void* xw, void* xout, float xeps, tfp8b_stream_t stream) {
    GemvSetup g;
    const int rc = gemv_setup(g, x_dtype, codes, scale, scale_kind, bias, y_dtype, M, N, K, G, fmt, xmode, true);
    if (rc != TFP8B_OK) return rc;
    return gemv_run(g, x, y, flags, xa, xb, xw, xout, xeps, stream);
}

// ------------------------------------------------------------------ prepared launches
struct tfp8b_gemv_plan {
    int max_M, device;
    GemvSetup by_m[9];          // by_m[M] for 1 <= M <= max_M (the weight tensor map is the same in all)
};

extern "C" int tfp8b_gemv_plan_create(tfp8b_gemv_plan** plan, int x_dtype, const uint8_t* codes, const void* scale,
                                      int scale_kind, const float* bias, int y_dtype, int max_M, int N, int K, int G, int fmt) {
    TFP8B_REQUIRE(plan, TFP8B_ERR_INVALID, "tfp8b_gemv_plan_create: null plan pointer");
    *plan = nullptr;
    TFP8B_REQUIRE(max_M >= 1 && max_M <= 8 && N >= 1, TFP8B_ERR_INVALID, "tfp8b_gemv_plan_create: 1 <= max_M <= 8 and N >= 1 (max_M=%d N=%d)",
                  max_M, N);
    tfp8b_gemv_plan* pl = static_cast<tfp8b_gemv_plan*>(calloc(1, sizeof(tfp8b_gemv_plan)));
    TFP8B_REQUIRE(pl, TFP8B_ERR_INVALID, "tfp8b_gemv_plan_create: out of host memory");
    pl->max_M = max_M;
    for (int M = 1; M <= max_M; ++M) {
        const int rc = gemv_setup(pl->by_m[M], x_dtype, codes, scale, scale_kind, bias, y_dtype, M, N, K, G, fmt, 0, true);
        if (rc != TFP8B_OK) { free(pl); return rc; }
    }
    cudaError_t e = cudaGetDevice(&pl->device);
    if (e != cudaSuccess) { free(pl); return cuda_fail(e, "cudaGetDevice"); }
    *plan = pl;
    return TFP8B_OK;
}

extern "C" int tfp8b_gemv_plan_run(const tfp8b_gemv_plan* plan, const void* x, void* y, int M, unsigned int flags,
                                   tfp8b_stream_t stream) {
    TFP8B_REQUIRE(plan, TFP8B_ERR_INVALID, "tfp8b_gemv_plan_run: null plan");
    if (M == 0) return TFP8B_OK;
    TFP8B_REQUIRE(M >= 1 && M <= plan->max_M, TFP8B_ERR_UNSUPPORTED, "tfp8b_gemv_plan_run: M=%d outside 1..%d", M, plan->max_M);
    return gemv_run(plan->by_m[M], x, y, flags, nullptr, nullptr, nullptr, nullptr, 0.f, stream);
}

extern "C" void tfp8b_gemv_plan_destroy(tfp8b_gemv_plan* plan) { free(plan); }
