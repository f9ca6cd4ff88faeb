// Decode GEMV for 1 <= M <= 8 activation rows (kernel a).
//
//   y[m,n] = sum_g scale[n,g] * sum_{k in g} x[m,k] * dec(codes[n,k]) + bias[n]
//
// The weight stream is the whole cost (N*K bytes against M*K + M*N elements of activations), so
// the kernel is built around keeping HBM busy:
//   * one CTA owns 16 consecutive weight rows and walks K in stages of 1024 codes;
//   * a producer warp moves each stage with 1-D bulk async copies (cp.async.bulk, 16 row copies
//     + M activation-row copies) into a ring of shared-memory stages, completion counted on an
//     mbarrier -- no registers are held for data in flight, and every byte of a row is requested
//     in large contiguous pieces with an evict-first L2 policy;
//   * eight consumer warps each take a 128-code slice of the stage: 128-bit shared loads, four
//     codes of a 32-bit word decoded with byte-permute / shift / mask bit moves to packed
//     f16x2 (or bf16x2), and the products are taken on the tensor cores with
//     mma.sync.m16n8k16 (16 weight rows x 8 activation rows, FP32 accumulate). At M = 8 the FP32
//     FMA pipe could not keep up with the byte rate of HBM3e; the MMA makes M irrelevant.
//   * x is consumed in its own type: f16 -> f16 MMA, bf16 -> bf16 MMA against bf16-decoded
//     weights (every FP8 value is exact in both), f32 -> split into three bf16 terms (24
//     mantissa bits) and three MMAs, so nothing is rounded before the FP32 accumulation.
//   * per-K-group scales are applied in FP32 to the partial sum of each group (exact for any
//     scale value), per-channel scales once at the end.
//   * the eight partial sums are added in a fixed order through shared memory: results are
//     deterministic and identical from call to call.
// All mbarrier waits are bounded; a wait that runs out sets a status bit and ends the CTA.
#include "common.cuh"

namespace tfp8b {

constexpr int GV_ROWS = 16;                      // weight rows per CTA (the MMA's M)
constexpr int GV_WARPS = 8;                      // consumer warps
constexpr int GV_THREADS = (GV_WARPS + 1) * 32;  // + one producer warp
constexpr int GV_KS = 1024;                      // codes of K per stage
constexpr int GV_WK = GV_KS / GV_WARPS;          // codes of K per warp per stage
constexpr int GV_MAX_STAGES = 8;
constexpr int GV_HEADER = 128 + GV_WARPS * GV_ROWS * 8 * 4;   // barriers + reduction buffer
constexpr int GV_SMEM_TARGET = 74 * 1024;        // per CTA, so that three CTAs share an SM

struct GemvParams {
    const void* x;
    const uint8_t* w;
    const void* scale;
    const float* bias;
    void* y;
    int M, N, K, G, scale_kind, y_dt;
    int nstages, wpitch, xpitch, stage_bytes;
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
// activations of row m. xq points at this lane's activations for the step.
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

// A 64-code block of the stage: lane (g, tig) takes the 16 codes at k = kofs + 16*tig of rows g
// and g+8 and the matching 16 activations of row m. MASK: the block is only half inside K (K is a
// multiple of 32), lanes with tig >= 2 contribute zeros.
template <typename XT, int FMT, bool MASK>
__device__ __forceinline__ void block64(float c[4], const uint8_t* wst, const uint8_t* xst, int wpitch, int xpitch,
                                        int g, int tig, int mrow, int kofs, int klen) {
    const int ko = kofs + tig * 16;
    uint4 wa = *reinterpret_cast<const uint4*>(wst + g * wpitch + ko);
    uint4 wb = *reinterpret_cast<const uint4*>(wst + (g + 8) * wpitch + ko);
    constexpr int XW = sizeof(XT) == 4 ? 16 : 8;           // 32-bit words of x per lane per block
    uint32_t xr[XW];
    const uint4* xp = reinterpret_cast<const uint4*>(xst + mrow * xpitch + ko * static_cast<int>(sizeof(XT)));
#pragma unroll
    for (int i = 0; i < XW / 4; ++i) {
        uint4 v = xp[i];
        xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
    }
    if (MASK && ko >= klen) {
        wa = make_uint4(0, 0, 0, 0); wb = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < XW; ++i) xr[i] = 0u;
    }
    const uint32_t was[4] = {wa.x, wa.y, wa.z, wa.w}, wbs[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) mma_step<XT, FMT>(c, was[j], wbs[j], &xr[j * (XW / 4)]);
}

// A 32-code block (32-wide scale groups): lane (g, tig) takes 8 codes at k = kofs + 8*tig.
template <typename XT, int FMT>
__device__ __forceinline__ void block32(float c[4], const uint8_t* wst, const uint8_t* xst, int wpitch, int xpitch,
                                        int g, int tig, int mrow, int kofs) {
    const int ko = kofs + tig * 8;
    uint2 wa = *reinterpret_cast<const uint2*>(wst + g * wpitch + ko);
    uint2 wb = *reinterpret_cast<const uint2*>(wst + (g + 8) * wpitch + ko);
    constexpr int XW = sizeof(XT) == 4 ? 8 : 4;
    uint32_t xr[XW];
    const uint4* xp = reinterpret_cast<const uint4*>(xst + mrow * xpitch + ko * static_cast<int>(sizeof(XT)));
#pragma unroll
    for (int i = 0; i < XW / 4; ++i) {
        uint4 v = xp[i];
        xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
    }
    mma_step<XT, FMT>(c, wa.x, wb.x, &xr[0]);
    mma_step<XT, FMT>(c, wa.y, wb.y, &xr[XW / 2]);
}

// SMODE 0: one scale per output channel (applied once, at the end)
//       1: K-groups that are multiples of 64 (applied per 64-code block)
//       2: K-groups that are multiples of 32 only (32-code blocks)
template <typename XT, int FMT, int SMODE>
__global__ void __launch_bounds__(GV_THREADS) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);               // full[0..7], empty[8..15]
    float* red = reinterpret_cast<float*>(smem + 128);                // [warp][row][m]
    uint8_t* stages = smem + GV_HEADER;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * GV_ROWS;
    const int S = p.nstages;
    const int nchunks = (p.K + GV_KS - 1) / GV_KS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[GV_MAX_STAGES + s]), GV_WARPS);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    if (warp == GV_WARPS) {
        // ---------------------------------------------------------------- producer warp
        const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
        const int row = min(n0 + (lane & 15), p.N - 1);                // N tail: re-read the last row
        const uint8_t* wsrc = p.w + static_cast<size_t>(row) * p.K;
        const int xm = lane - 16;
        const uint8_t* xsrc = reinterpret_cast<const uint8_t*>(p.x) + static_cast<size_t>(max(xm, 0)) * p.K * sizeof(XT);
        for (int c = 0; c < nchunks; ++c) {
            const int slot = c % S;
            if (c >= S && !mbar_wait(smem_u32(&bars[GV_MAX_STAGES + slot]), ((c / S) - 1) & 1, STATUS_GEMV_WAIT)) break;
            const int k0 = c * GV_KS, klen = min(GV_KS, p.K - k0);
            const uint32_t full = smem_u32(&bars[slot]);
            uint8_t* wst = stages + static_cast<size_t>(slot) * p.stage_bytes;
            uint8_t* xst = wst + GV_ROWS * p.wpitch;
            if (lane == 0) mbar_expect_tx(full, static_cast<uint32_t>(GV_ROWS * klen + p.M * klen * static_cast<int>(sizeof(XT))));
            __syncwarp();
            if (lane < 16) bulk_g2s(smem_u32(wst + lane * p.wpitch), wsrc + k0, klen, full, pol_w);
            else if (xm < p.M) bulk_g2s(smem_u32(xst + xm * p.xpitch), xsrc + static_cast<size_t>(k0) * sizeof(XT),
                                        klen * static_cast<int>(sizeof(XT)), full, pol_x);
        }
    } else {
        // ---------------------------------------------------------------- consumer warps
        const int g = lane >> 2, tig = lane & 3;
        const int mrow = min(g, p.M - 1);
        const int ng = p.K / p.G;
        const size_t srow_a = static_cast<size_t>(min(n0 + g, p.N - 1)) * ng;
        const size_t srow_b = static_cast<size_t>(min(n0 + g + 8, p.N - 1)) * ng;
        constexpr int BLK = SMODE == 2 ? 32 : 64;
        constexpr int NB = GV_WK / BLK;
        const int kw = warp * GV_WK;
        for (int c = 0; c < nchunks; ++c) {
            const int slot = c % S;
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
            if (!mbar_wait(smem_u32(&bars[slot]), (c / S) & 1, STATUS_GEMV_WAIT)) break;
            const uint8_t* wst = stages + static_cast<size_t>(slot) * p.stage_bytes;
            const uint8_t* xst = wst + GV_ROWS * p.wpitch;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const int kofs = kw + b * BLK;
                if (kofs < klen) {
                    if (SMODE == 0) {
                        if (kofs + 64 <= klen) block64<XT, FMT, false>(acc, wst, xst, p.wpitch, p.xpitch, g, tig, mrow, kofs, klen);
                        else block64<XT, FMT, true>(acc, wst, xst, p.wpitch, p.xpitch, g, tig, mrow, kofs, klen);
                    } else {
                        float t[4] = {0.f, 0.f, 0.f, 0.f};
                        if (SMODE == 2) block32<XT, FMT>(t, wst, xst, p.wpitch, p.xpitch, g, tig, mrow, kofs);
                        else if (kofs + 64 <= klen) block64<XT, FMT, false>(t, wst, xst, p.wpitch, p.xpitch, g, tig, mrow, kofs, klen);
                        else block64<XT, FMT, true>(t, wst, xst, p.wpitch, p.xpitch, g, tig, mrow, kofs, klen);
                        acc[0] = fmaf(t[0], sa[b], acc[0]); acc[1] = fmaf(t[1], sa[b], acc[1]);
                        acc[2] = fmaf(t[2], sb[b], acc[2]); acc[3] = fmaf(t[3], sb[b], acc[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[GV_MAX_STAGES + slot]));
        }
        float* r = red + warp * (GV_ROWS * 8);
        r[g * 8 + 2 * tig] = acc[0];
        r[g * 8 + 2 * tig + 1] = acc[1];
        r[(g + 8) * 8 + 2 * tig] = acc[2];
        r[(g + 8) * 8 + 2 * tig + 1] = acc[3];
    }
    __syncthreads();

    // ---------------------------------------------------------------- fixed-order reduction + epilogue
    if (threadIdx.x < GV_ROWS * 8) {
        const int row = threadIdx.x & 15, m = threadIdx.x >> 4;
        const int n = n0 + row;
        if (n < p.N && m < p.M) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < GV_WARPS; ++w) v += red[w * (GV_ROWS * 8) + row * 8 + m];
            const float b = p.bias ? p.bias[n] : 0.f;
            if (SMODE == 0) v = fmaf(v, load_scale(p.scale, n, p.scale_kind), b);
            else v += b;
            store_dt(p.y, static_cast<size_t>(m) * p.N + n, v, p.y_dt);
        }
    }
}

template <typename XT, int FMT, int SMODE>
static int launch_gemv(const GemvParams& p, size_t smem, cudaStream_t st) {
    // The opt-in to more than 48 KB of dynamic shared memory is per device and per kernel.
    static unsigned long long configured = 0ull;        // bit d set: done on device d
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev >= 64 || !((configured >> dev) & 1ull)) {
        e = cudaFuncSetAttribute(gemv_kernel<XT, FMT, SMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemv)");
        if (dev < 64) __atomic_fetch_or(&configured, 1ull << dev, __ATOMIC_RELAXED);
    }
    const int grid = (p.N + GV_ROWS - 1) / GV_ROWS;
    gemv_kernel<XT, FMT, SMODE><<<grid, GV_THREADS, smem, st>>>(p);
    TFP8B_LAUNCH_CHECK("tfp8b_gemv");
    return TFP8B_OK;
}

template <typename XT>
static int dispatch_gemv(const GemvParams& p, int fmt, int smode, size_t smem, cudaStream_t st) {
#define GV_CASE(F, S) if (fmt == F && smode == S) return launch_gemv<XT, F, S>(p, smem, st)
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
    TFP8B_REQUIRE(M >= 0 && N >= 0 && K > 0 && G > 0, TFP8B_ERR_INVALID, "tfp8b_gemv: bad size M=%d N=%d K=%d G=%d", M, N, K, G);
    TFP8B_REQUIRE(x_dtype >= 0 && x_dtype <= 2 && y_dtype >= 0 && y_dtype <= 2, TFP8B_ERR_INVALID, "tfp8b_gemv: bad dtype");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_gemv: bad fmt %d", fmt);
    TFP8B_REQUIRE(scale_kind == TFP8B_SCALE_F32 || scale_kind == TFP8B_SCALE_UE8M0, TFP8B_ERR_INVALID,
                  "tfp8b_gemv: bad scale_kind %d", scale_kind);
    TFP8B_REQUIRE(M <= 8, TFP8B_ERR_UNSUPPORTED, "tfp8b_gemv: M=%d > 8, use tfp8b_gemm", M);
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x && codes && scale && y, TFP8B_ERR_INVALID, "tfp8b_gemv: null pointer");
    TFP8B_REQUIRE(K % 32 == 0 && G % 32 == 0 && K % G == 0, TFP8B_ERR_UNSUPPORTED,
                  "tfp8b_gemv: need K %% 32 == 0, G %% 32 == 0, K %% G == 0 (K=%d G=%d)", K, G);
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(codes)) & 15u) == 0, TFP8B_ERR_INVALID,
                  "tfp8b_gemv: x and codes must be 16-byte aligned");
    const int smode = G == K ? 0 : (G % 64 == 0 ? 1 : 2);
    const int xsz = dtype_size(x_dtype);
    GemvParams p;
    p.x = x; p.w = codes; p.scale = scale; p.bias = bias; p.y = y;
    p.M = M; p.N = N; p.K = K; p.G = G; p.scale_kind = scale_kind; p.y_dt = y_dtype;
    // Row pitches that keep the 128-bit (64-code blocks) or 64-bit (32-code blocks) shared loads
    // of a quarter / half warp on distinct banks.
    p.wpitch = GV_KS + (smode == 2 ? 32 : 64);
    p.xpitch = GV_KS * xsz + (smode == 2 ? 64 : 16);
    p.stage_bytes = (GV_ROWS * p.wpitch + M * p.xpitch + 127) & ~127;
    const int nchunks = (K + GV_KS - 1) / GV_KS;
    int S = (GV_SMEM_TARGET - GV_HEADER) / p.stage_bytes;
    S = S < 2 ? 2 : (S > GV_MAX_STAGES ? GV_MAX_STAGES : S);
    if (S > nchunks) S = nchunks;
    p.nstages = S;
    const size_t smem = GV_HEADER + static_cast<size_t>(S) * p.stage_bytes;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == TFP8B_F16) return dispatch_gemv<__half>(p, fmt, smode, smem, st);
    if (x_dtype == TFP8B_BF16) return dispatch_gemv<__nv_bfloat16>(p, fmt, smode, smem, st);
    return dispatch_gemv<float>(p, fmt, smode, smem, st);
}
