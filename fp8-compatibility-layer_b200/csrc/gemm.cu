// Tile GEMM on prepared fp16 activations (kernel b):
//
//   y[m,n] = xs[m] * smax[n] * sum_k x16[m,k] * (dec(codes[n,k]) * scale[n,k/G] / smax[n]) + bias[n]
//
// Computed transposed, D[n, m], so that the 128 rows of the tcgen05 MMA are WEIGHT rows: a CTA
// decodes each FP8 tile once and multiplies it against up to 256 activation rows, and small M
// (16..128) simply uses a narrower MMA instead of padding the 128-row dimension.
//
// Per CTA: 128 weight rows x BN activation rows (BN = 16..256), K walked in 64-wide blocks through
// a ring of shared-memory stages:
//   warp 0      TMA producer: one 2-D tiled load of the raw FP8 tile (128 x 64 bytes) and one of
//               the activation tile (BN x 64 fp16, 128-byte swizzle) per stage, no multicast;
//   warps 2..5  decode: 16 codes per thread per step by byte-permute/shift/mask bit moves to
//               fp16, group-scale ratio folded in (FP32 multiply, one fp16 rounding -- exact for
//               power-of-two scales), written in the 128-byte-swizzled K-major layout the MMA
//               reads; fence.proxy.async, then an mbarrier arrive;
//   warp 1      one thread issues tcgen05.mma (kind::f16, M=128, N=BN, K=16) four times per
//               stage, accumulating in tensor memory, and tcgen05.commit frees the stage;
//   warps 2..5  epilogue: tcgen05.ld the FP32 accumulators, apply smax[n], xs[m], bias[n], round
//               once to the output type and store (32 lanes = 32 consecutive n per m).
// No fp16 copy of the weights ever exists outside shared memory. Every mbarrier wait is bounded.
#include "common.cuh"

namespace tfp8b {

constexpr int GM_BM = 128;          // weight rows per CTA = UMMA M = TMEM lanes
constexpr int GM_BK = 64;           // K per stage: one 128-byte swizzle atom of fp16
constexpr int GM_THREADS = 192;
constexpr int GM_MAX_STAGES = 8;
constexpr int GM_HEADER = 2048;     // barriers, TMEM base, per-row scale maxima
constexpr int GM_A_BYTES = GM_BM * GM_BK * 2;    // decoded fp16 tile
constexpr int GM_RAW_BYTES = GM_BM * GM_BK;      // raw FP8 tile
constexpr int GM_SMEM_MAX = 232448;              // 227 KB opt-in limit per CTA

struct GemmParams {
    const float* xs;
    const void* scale;
    const float* bias;
    void* y;
    int M, N, K, G, scale_kind, y_dt;
    int BN, nstages, stage_bytes, tmem_cols;
};

struct GemmHeader {
    uint64_t full_raw[GM_MAX_STAGES];
    uint64_t full_a[GM_MAX_STAGES];
    uint64_t empty[GM_MAX_STAGES];
    uint64_t acc_full;
    uint32_t tmem_base;
    uint32_t pad;
    float smax[GM_BM];      // per weight row: max_g scale[n,g] (the scale itself for one group)
    float binv[GM_BM];      // 1 / smax (0 when smax == 0)
};
static_assert(sizeof(GemmHeader) <= GM_HEADER, "header too large");

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

// ------------------------------------------------------------------ the kernel
template <int FMT>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment of the stage buffers is required by the swizzled layouts.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    GemmHeader* hd = reinterpret_cast<GemmHeader*>(smem);
    uint8_t* stages = smem + GM_HEADER;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * p.BN;        // activation-row tile (fast grid dimension: CTAs that
    const int n0 = blockIdx.y * GM_BM;       // run together share one weight stripe through L2)
    const int S = p.nstages;
    const int nkb = (p.K + GM_BK - 1) / GM_BK;
    const int x_bytes = p.BN * GM_BK * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(smem_u32(&hd->full_raw[s]), 1);
            mbar_init(smem_u32(&hd->full_a[s]), 4);
            mbar_init(smem_u32(&hd->empty[s]), 1);
        }
        mbar_init(smem_u32(&hd->acc_full), 1);
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
    const uint32_t tmem_acc = hd->tmem_base;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            // One activation tile only: the weight stripe is read once, keep it out of L2's way.
            // Several tiles: the CTAs of the other tiles read the same stripe from L2 next.
            const uint64_t pol_w = gridDim.x == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
            const uint64_t pol_x = l2_policy_evict_last();
            for (int kb = 0; kb < nkb; ++kb) {
                const int slot = kb % S;
                if (kb >= S && !mbar_wait(smem_u32(&hd->empty[slot]), ((kb / S) - 1) & 1, STATUS_GEMM_WAIT)) break;
                uint8_t* st = stages + static_cast<size_t>(slot) * p.stage_bytes;
                const uint32_t bar = smem_u32(&hd->full_raw[slot]);
                mbar_expect_tx(bar, static_cast<uint32_t>(GM_RAW_BYTES + x_bytes));
                tma_load_2d(smem_u32(st + GM_A_BYTES), &tm_x, kb * GM_BK, m0, bar, pol_x);
                tma_load_2d(smem_u32(st + GM_A_BYTES + x_bytes), &tm_w, kb * GM_BK, n0, bar, pol_w);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // D fp32, A/B fp16, both K-major, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(p.BN >> 3) << 17) | (static_cast<uint32_t>(GM_BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int slot = kb % S;
                const uint32_t par = (kb / S) & 1;
                ok = mbar_wait(smem_u32(&hd->full_raw[slot]), par, STATUS_GEMM_WAIT) &&
                     mbar_wait(smem_u32(&hd->full_a[slot]), par, STATUS_GEMM_WAIT);
                if (!ok) break;
                tc_fence_after();
                uint8_t* st = stages + static_cast<size_t>(slot) * p.stage_bytes;
                const uint64_t da = umma_desc_sw128(smem_u32(st));
                const uint64_t db = umma_desc_sw128(smem_u32(st + GM_A_BYTES));
#pragma unroll
                for (int kk = 0; kk < GM_BK / 16; ++kk)
                    tc_mma_f16(tmem_acc, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                tc_commit(smem_u32(&hd->empty[slot]));
            }
            if (ok) tc_commit(smem_u32(&hd->acc_full));
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- decode warps, then epilogue
        const int td = threadIdx.x - 64;             // 0..127
        const int ng = p.K / p.G;
        {   // per-row scale maximum for TMEM lane td (row n0 + td)
            const int n = min(n0 + td, p.N - 1);
            float mx = 0.f;
            if (ng == 1) {
                mx = load_scale(p.scale, n, p.scale_kind);
            } else {
                for (int gi = 0; gi < ng; ++gi) mx = fmaxf(mx, load_scale(p.scale, static_cast<size_t>(n) * ng + gi, p.scale_kind));
            }
            hd->smax[td] = mx;
            hd->binv[td] = mx > 0.f ? 1.f / mx : 0.f;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");

        const int c = td & 3;                        // 16-code chunk of the 64-wide K block
        int rows[4];
        size_t srow[4];
        float binv[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            rows[it] = (td >> 2) + 32 * it;
            srow[it] = static_cast<size_t>(min(n0 + rows[it], p.N - 1)) * ng;
            binv[it] = hd->binv[rows[it]];
        }
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb) {
            const int slot = kb % S;
            float ratio[4] = {1.f, 1.f, 1.f, 1.f};
            if (ng > 1) {
                const int gi = min((kb * GM_BK + c * 16) / p.G, ng - 1);
#pragma unroll
                for (int it = 0; it < 4; ++it) ratio[it] = load_scale(p.scale, srow[it] + gi, p.scale_kind) * binv[it];
            }
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->full_raw[slot]), (kb / S) & 1, STATUS_GEMM_WAIT));
            if (!ok) break;
            uint8_t* st = stages + static_cast<size_t>(slot) * p.stage_bytes;
            const uint8_t* raw = st + GM_A_BYTES + x_bytes;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int r = rows[it];
                const uint4 q = *reinterpret_cast<const uint4*>(raw + r * GM_BK + c * 16);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                uint32_t h[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) dec4<FMT, false>(w[j], h[2 * j], h[2 * j + 1]);
                if (ratio[it] != 1.f) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float2 f = __half22float2(*reinterpret_cast<__half2*>(&h[j]));
                        __half2 o = __floats2half2_rn(f.x * ratio[it], f.y * ratio[it]);
                        h[j] = *reinterpret_cast<uint32_t*>(&o);
                    }
                }
                uint8_t* arow = st + r * 128;
                *reinterpret_cast<uint4*>(arow + (((2 * c) ^ (r & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4*>(arow + (((2 * c + 1) ^ (r & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
            }
            fence_proxy_async_smem();        // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&hd->full_a[slot]));
        }

        // ---------------------------------------------------------------- epilogue
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&hd->acc_full), 0, STATUS_GEMM_WAIT));
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3;                       // TMEM lanes this warp may read
            const int row = quarter * 32 + lane;
            const int n = n0 + row;
            const float sm = hd->smax[row];
            const float b = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            for (int col = 0; col < p.BN; col += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + col, v);
                tmem_ld_wait();
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + col + j;
                        if (m < p.M)
                            store_dt(p.y, static_cast<size_t>(m) * p.N + n, fmaf(__uint_as_float(v[j]) * sm, p.xs[m], b), p.y_dt);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_acc, static_cast<uint32_t>(p.tmem_cols));
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

static int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                       uint64_t outer, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return TFP8B_ERR_CUDA; }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r)); return TFP8B_ERR_CUDA; }
    return TFP8B_OK;
}

template <int FMT>
static int launch_gemm(const CUtensorMap& tw, const CUtensorMap& tx, const GemmParams& p, size_t smem, cudaStream_t st) {
    static unsigned long long configured = 0ull;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev >= 64 || !((configured >> dev) & 1ull)) {
        e = cudaFuncSetAttribute(gemm_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, GM_SMEM_MAX);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm)");
        if (dev < 64) __atomic_fetch_or(&configured, 1ull << dev, __ATOMIC_RELAXED);
    }
    dim3 grid((p.M + p.BN - 1) / p.BN, (p.N + GM_BM - 1) / GM_BM);
    gemm_kernel<FMT><<<grid, GM_THREADS, smem, st>>>(tw, tx, p);
    TFP8B_LAUNCH_CHECK("tfp8b_gemm");
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
    TFP8B_REQUIRE(M >= 0 && N >= 0 && K > 0 && G > 0, TFP8B_ERR_INVALID, "tfp8b_gemm: bad size M=%d N=%d K=%d G=%d", M, N, K, G);
    TFP8B_REQUIRE(y_dtype >= 0 && y_dtype <= 2, TFP8B_ERR_INVALID, "tfp8b_gemm: bad dtype");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_gemm: bad fmt %d", fmt);
    TFP8B_REQUIRE(scale_kind == TFP8B_SCALE_F32 || scale_kind == TFP8B_SCALE_UE8M0, TFP8B_ERR_INVALID,
                  "tfp8b_gemm: bad scale_kind %d", scale_kind);
    if (M == 0 || N == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x16 && xs && codes && scale && y, TFP8B_ERR_INVALID, "tfp8b_gemm: null pointer");
    TFP8B_REQUIRE(K % 32 == 0 && G % 32 == 0 && K % G == 0, TFP8B_ERR_UNSUPPORTED,
                  "tfp8b_gemm: need K %% 32 == 0, G %% 32 == 0, K %% G == 0 (K=%d G=%d)", K, G);
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(x16) | reinterpret_cast<uintptr_t>(codes)) & 15u) == 0, TFP8B_ERR_INVALID,
                  "tfp8b_gemm: x16 and codes must be 16-byte aligned");
    GemmParams p;
    p.xs = xs; p.scale = scale; p.bias = bias; p.y = y;
    p.M = M; p.N = N; p.K = K; p.G = G; p.scale_kind = scale_kind; p.y_dt = y_dtype;
    int bn = 16;
    while (bn < M && bn < 256) bn <<= 1;
    p.BN = bn;
    p.tmem_cols = bn < 32 ? 32 : bn;
    p.stage_bytes = GM_A_BYTES + bn * GM_BK * 2 + GM_RAW_BYTES;
    const int nkb = (K + GM_BK - 1) / GM_BK;
    int S = (GM_SMEM_MAX - 1024 - GM_HEADER) / p.stage_bytes;
    S = S > GM_MAX_STAGES ? GM_MAX_STAGES : S;
    if (S > nkb) S = nkb;
    p.nstages = S;
    const size_t smem = 1024 + GM_HEADER + static_cast<size_t>(S) * p.stage_bytes;

    CUtensorMap tw, tx;
    int rc = make_map_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, codes, static_cast<uint64_t>(K), static_cast<uint64_t>(N),
                         GM_BK, GM_BM, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != TFP8B_OK) return rc;
    rc = make_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                     GM_BK, static_cast<uint32_t>(bn), CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != TFP8B_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (fmt == TFP8B_E4M3FN) return launch_gemm<TFP8B_E4M3FN>(tw, tx, p, smem, st);
    return launch_gemm<TFP8B_E5M2>(tw, tx, p, smem, st);
}
