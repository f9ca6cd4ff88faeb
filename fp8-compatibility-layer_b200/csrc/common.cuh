// Shared device helpers for the tfp8b kernels (sm_100a): FP8 bit decode/encode, mbarrier /
// bulk-copy / TMA / tcgen05 PTX wrappers, and the host-side error plumbing of the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../../include/tfp8b.h"

namespace tfp8b {

// ------------------------------------------------------------------ host-side error plumbing
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define TFP8B_REQUIRE(cond, code, ...)      \
    do {                                    \
        if (!(cond)) {                      \
            ::tfp8b::set_error(__VA_ARGS__); \
            return (code);                  \
        }                                   \
    } while (0)

#define TFP8B_LAUNCH_CHECK(what)                                      \
    do {                                                              \
        cudaError_t e__ = cudaGetLastError();                         \
        if (e__ != cudaSuccess) return ::tfp8b::cuda_fail(e__, what); \
    } while (0)

// Device-side status word, one per translation unit (the library is built without relocatable
// device code): kernels OR a bit in when a bounded wait runs out; each .cu file that has such
// waits exports a reader that tfp8b_device_status() combines.
static __device__ unsigned int g_status;
constexpr unsigned STATUS_GEMV_WAIT = 1u, STATUS_GEMM_WAIT = 2u, STATUS_GLUE_WAIT = 4u, STATUS_GLUE_POS = 8u;
int read_and_clear_status(unsigned int* word_on_device, unsigned int* out, cudaStream_t st);

// Host: fills a tiled tensor map (cuTensorMapEncodeTiled, fetched from the driver at first use).
// dims / box have `rank` entries (innermost first), strides_bytes rank - 1 (dimension 1 upwards).
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const cuuint64_t* dims,
                      const cuuint64_t* strides_bytes, const cuuint32_t* box, CUtensorMapSwizzle swizzle);

// ------------------------------------------------------------------ small utilities
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

template <typename T> struct dtype_of;
template <> struct dtype_of<__half> { static constexpr int id = TFP8B_F16; };
template <> struct dtype_of<__nv_bfloat16> { static constexpr int id = TFP8B_BF16; };
template <> struct dtype_of<float> { static constexpr int id = TFP8B_F32; };

__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == TFP8B_F32 ? 4 : 2; }

__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }

__device__ __forceinline__ void store_as(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_as(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void store_as(float* p, float v) { *p = v; }

// y[i] = v in a runtime-selected element type (used by epilogues that are not templated on it).
__device__ __forceinline__ void store_dt(void* y, size_t i, float v, int dt) {
    if (dt == TFP8B_F16) reinterpret_cast<__half*>(y)[i] = __float2half_rn(v);
    else if (dt == TFP8B_BF16) reinterpret_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(y)[i] = v;
}

// Weight scale -> float. UE8M0 byte b is 2^(b-127): the float32 bit pattern b<<23, except b == 0
// (2^-127, a float32 subnormal) and b == 255 (NaN).
__device__ __forceinline__ float ue8m0_to_f32(uint32_t b) {
    uint32_t u = b << 23;
    if (b == 0u) u = 0x00400000u;
    if (b == 255u) u = 0x7FC00000u;
    return __uint_as_float(u);
}
__device__ __forceinline__ float load_scale(const void* s, size_t i, int kind) {
    return kind == TFP8B_SCALE_UE8M0 ? ue8m0_to_f32(reinterpret_cast<const uint8_t*>(s)[i])
                                     : reinterpret_cast<const float*>(s)[i];
}

// ------------------------------------------------------------------ FP8 decode
// Two codes -> one packed f16x2 / bf16x2 word, exact for every code (subnormals, -0, NaN, inf).
//
// E5M2 -> f16 is a byte move (same exponent bias): the code is the high byte of the half.
// E4M3FN -> f16 uses the conversion instruction cvt.rn.f16x2.e4m3x2. Measured on B200 over all
// SMs (decode only, codes per clock per SM; HBM3e delivers about 23 bytes per clock per SM):
//     byte-permute / shift / mask / multiply bit moves, NaN-exact   23.8
//     the same without the NaN fix-up                               29.1
//     cvt.rn.f16x2.e4m3x2                                           84.1
//     E5M2 byte move                                                99.3
// so the bit-move decode alone would eat the whole issue budget of a bandwidth-bound kernel;
// it is kept below (TFP8B_DECODE_BITMOVES) as the definition the conversion is tested against.
// bf16 targets go through f16 -> f32 -> bf16x2 (all exact: every FP8 value fits bf16).
template <int FMT>
__device__ __forceinline__ uint32_t dec2_f16_bitmoves(uint32_t q) {
    // q: one code in the HIGH byte of each 16-bit lane (c << 8), low bytes zero.
    //   E4M3FN: s eeee mmm -> s 0eeee mmm0000000 (shift 1), then * 2^8 rebiases 7 -> 15 and makes
    //   the subnormals exact; 0x7F / 0xFF (all magnitude bits set) get exponent 11111 first = NaN.
    if (FMT == TFP8B_E5M2) return q;
    uint32_t mag = (q >> 1) & 0x3F803F80u;
    uint32_t nan = (mag + 0x00800080u) & 0x40004000u;
    mag |= nan;
    __half2 h = __hmul2(*reinterpret_cast<__half2*>(&mag), __half2half2(__ushort_as_half(0x5C00)));
    return *reinterpret_cast<uint32_t*>(&h) | (q & 0x80008000u);
}

// pair: two codes in the low 16 bits (c0 low byte, c1 high byte) -> f16x2 {c0, c1}
template <int FMT>
__device__ __forceinline__ uint32_t dec2_f16(uint32_t pair16) {
#ifdef TFP8B_DECODE_BITMOVES
    return dec2_f16_bitmoves<FMT>(__byte_perm(pair16, 0u, 0x1404));
#else
    if (FMT == TFP8B_E5M2) return __byte_perm(pair16, 0u, 0x1404);        // (c1 << 24) | (c0 << 8)
    uint32_t out;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(out) : "h"(static_cast<unsigned short>(pair16)));
    return out;
#endif
}

__device__ __forceinline__ uint32_t f16x2_to_bf16x2(uint32_t h) {
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
    __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    return *reinterpret_cast<uint32_t*>(&b);
}

// Four codes of one 32-bit word (c0 in the low byte) -> two packed pairs {c0,c1}, {c2,c3}.
template <int FMT, bool BF16>
__device__ __forceinline__ void dec4(uint32_t w, uint32_t& p01, uint32_t& p23) {
#ifndef TFP8B_DECODE_BITMOVES
    if (FMT == TFP8B_E5M2) {
        p01 = __byte_perm(w, 0u, 0x1404);      // (c1 << 24) | (c0 << 8)
        p23 = __byte_perm(w, 0u, 0x3424);      // (c3 << 24) | (c2 << 8)
    } else
#endif
    {
        p01 = dec2_f16<FMT>(w & 0xFFFFu);
        p23 = dec2_f16<FMT>(w >> 16);
    }
    if (BF16) { p01 = f16x2_to_bf16x2(p01); p23 = f16x2_to_bf16x2(p23); }
}

// The same four codes -> two f16x2 words with the word split into its 16-bit halves INSIDE the asm
// block, so that no mask / shift instructions stand between the load and the two conversions.
// Measured per kernel: 3 % faster in the tile GEMM's decode warps, 0.5 % slower in the GEMV's
// consumer loop (which is why both forms exist). fp16 output only.
template <int FMT>
__device__ __forceinline__ void dec4_split(uint32_t w, uint32_t& p01, uint32_t& p23) {
#ifndef TFP8B_DECODE_BITMOVES
    if (FMT == TFP8B_E4M3FN) {
        asm("{\n\t.reg .b16 lo, hi;\n\t"
            "mov.b32 {lo, hi}, %2;\n\t"
            "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
            "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
            : "=r"(p01), "=r"(p23) : "r"(w));
        return;
    }
#endif
    dec4<FMT, false>(w, p01, p23);
}

// ------------------------------------------------------------------ FP8 encode (exact, integer)
// float -> code: round to nearest even on the float's bit fields, saturate to the largest finite
// code (also for +-inf), NaN -> sign|0x7F (nan_mode CAST) or the format's canonical NaN.
//   EB/MB: exponent / mantissa bits, BIAS: exponent bias, TOP: largest finite code (0x7E / 0x7B).
template <int FMT>
__host__ __device__ __forceinline__ uint32_t encode1(float x, int nan_mode) {
    constexpr int MB = FMT == TFP8B_E4M3FN ? 3 : 2;
    constexpr int BIAS = FMT == TFP8B_E4M3FN ? 7 : 15;
    constexpr uint32_t TOP = FMT == TFP8B_E4M3FN ? 0x7Eu : 0x7Bu;
    constexpr uint32_t NAN_CANON = FMT == TFP8B_E4M3FN ? 0x7Fu : 0x7Eu;
    constexpr int EMIN = 1 - BIAS;                       // exponent of the smallest normal
#ifdef __CUDA_ARCH__
    const uint32_t u = __float_as_uint(x);
#else
    union { float f; uint32_t u; } cvt_; cvt_.f = x; const uint32_t u = cvt_.u;
#endif
    const uint32_t sign = (u >> 24) & 0x80u;
    const uint32_t ax = u & 0x7FFFFFFFu;
    if (ax > 0x7F800000u) return nan_mode == TFP8B_NAN_CANONICAL ? NAN_CANON : (sign | 0x7Fu);
    const int e = static_cast<int>(ax >> 23) - 127;      // unbiased float exponent (-127 for 0/sub)
    uint32_t code;
    if (e >= EMIN) {
        // normal target: keep MB mantissa bits, RNE on the 23-MB dropped bits; a mantissa carry
        // walks into the exponent field because the fields are adjacent.
        const uint32_t keep = ax >> (23 - MB);                        // exponent|mantissa, float bias
        const uint32_t rest = ax & ((1u << (23 - MB)) - 1u);
        const uint32_t half = 1u << (22 - MB);
        const uint32_t up = (rest > half) || (rest == half && (keep & 1u));
        const uint32_t r = keep + up;
        const int re = static_cast<int>(r >> MB) - 127 + BIAS;        // target exponent field
        code = (static_cast<uint32_t>(re) << MB) | (r & ((1u << MB) - 1u));
        if (re <= 0) code = 0;                                        // cannot happen for e >= EMIN
        if (code > TOP || re >= (1 << (7 - MB))) code = TOP;          // saturate (inf included)
    } else {
        // subnormal target: value = m * 2^(EMIN-MB); m = RNE(|x| * 2^(MB-EMIN)), 0 <= m <= 2^MB
        // (m == 2^MB is the smallest normal: the same bit pattern).
        const int shift = (EMIN - MB) - (e - 23);                     // bits to drop from the 24-bit significand
        if (e == -127 || shift > 25) {
            code = 0;                                                 // zero / float subnormal / far below half a step
        } else {
            const uint32_t sig = (ax & 0x7FFFFFu) | 0x800000u;
            const uint32_t keep = sig >> shift;
            const uint32_t rest = sig & ((1u << shift) - 1u);
            const uint32_t half = 1u << (shift - 1);
            code = keep + ((rest > half) || (rest == half && (keep & 1u)));
        }
    }
    return sign | code;
}

__host__ __device__ __forceinline__ uint32_t encode1(float x, int fmt, int nan_mode) {
    return fmt == TFP8B_E5M2 ? encode1<TFP8B_E5M2>(x, nan_mode) : encode1<TFP8B_E4M3FN>(x, nan_mode);
}

// Two floats -> two codes (lo in bits 0-7) by the conversion instruction: round to nearest even,
// saturate to the largest finite code (+-inf included). A NaN comes back as some NaN code of the
// format, never as a finite one, which is all `encode16` relies on.
template <int FMT>
__device__ __forceinline__ uint32_t enc2_hw(float lo, float hi) {
    unsigned short r;
    if (FMT == TFP8B_E4M3FN) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// Scale of a group from its largest magnitude, the rule of the reference's quantize_weight
// (tfp8/quantize.py:27-33): amax / fmax, at least the smallest normal float, rounded up to a power
// of two on request; 1 for an all-zero group.
__device__ __forceinline__ float scale_from_amax(float amax, float fmax, int pow2) {
    if (amax == 0.f) return 1.f;
    float s = fmaxf(__fdiv_rn(amax, fmax), FLT_MIN);
    if (pow2) {
        uint32_t u = __float_as_uint(s);
        if (u & 0x007FFFFFu) u = (u & 0x7F800000u) + 0x00800000u;   // next power of two
        s = __uint_as_float(u);
    }
    return s;
}

// ------------------------------------------------------------------ mbarrier / bulk copy
#ifdef __CUDACC__
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The same test, but the thread may be suspended by the hardware until the phase completes or
// `ns` nanoseconds have passed, instead of coming straight back: a waiting warp then costs no
// issue slots, which on an SM whose other warps are doing the work is the difference between
// polling and waiting (the tile GEMM at 16 rows spent more than two thirds of its issued
// instructions in polls).
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait: tests once, then waits in suspended polls of up to 20 us each and gives up after
// about two seconds of SM clock, records `status_bit` in the device status word and returns
// false. No wait in this library is unbounded, so a protocol error ends the kernel instead of
// hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned status_bit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait_suspend(bar, parity, 20000u)) return true;
        if (clock64() - t0 > (1ll << 32)) break;
    }
    atomicOr(&g_status, status_bit);
    return false;
}
// The same wait for a whole (converged) warp: one lane polls, the others sleep at the shuffle.
// 256 threads polling one mbarrier keep the shared-memory pipe busy for nothing.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, unsigned status_bit) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, status_bit) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_normal() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// 1-D bulk copy global -> shared of this CTA, completion counted in bytes on `bar`.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
// 2-D tiled TMA load (no multicast), coordinates in elements: c0 innermost.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy) : "memory");
}
// 3-D tiled TMA load (no multicast), coordinates in elements: c0 innermost.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy) : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its prologue now /
// wait until everything the previous kernel wrote is visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
#endif  // __CUDACC__

}  // namespace tfp8b
