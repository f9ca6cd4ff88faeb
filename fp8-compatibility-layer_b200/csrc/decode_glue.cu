// Small fused kernels for the decode step AROUND the FP8Linear layers of a Llama-style block (the
// reference's demo does these with a dozen eager torch kernels per layer, which on B200 cost
// more time than the FP8 GEMVs themselves):
//   rope_kv_store  rotary embedding of Q and K from the fused QKV projection, Q written
//                  head-major for the attention call, K and V written into the static KV cache
//                  at the tokens' positions -- one launch instead of ~16;
//   silu_mul       silu(gate) * up on the fused gate/up projection -- one launch instead of 2-3;
//   add_rmsnorm    residual += delta, then RMSNorm of the residual -- one launch instead of 2;
//   argmax         greedy token choice over the vocabulary, one CTA per row;
//   attn_decode    one-query attention over the static KV cache (grouped-query heads), the KV
//                  range split across CTAs and merged by a second small kernel;
//   rope_kv_store_fp8 / attn_decode_fp8  the same two over an FP8 KV cache (codes + one scale per
//                  token and KV head): half the cache, half the bytes an attention step reads.
// All are plain bandwidth- or latency-bound kernels on 16-bit activations. They are launched
// with programmatic stream serialization and release their dependents at once: the FP8 GEMV
// that follows starts streaming its weights while the helper is still running, and waits for
// it (griddepcontrol.wait) only before it reads the activations.
// A kernel launched that way is alive while its predecessor still writes, so nothing it reads
// is "read-only for the lifetime of the kernel": no pointer here is __restrict__ and nothing is
// loaded through the non-coherent path (__ldg / ld.global.nc). With them the compiler used that
// path for the FP8 cache's per-position scales, whose 128-byte lines are shared by 32 positions:
// a line cached when the previous token's step read it came back without the newest scale.
#include <stdlib.h>

#include "common.cuh"

namespace tfp8b {

template <typename T> struct pair_of;
template <> struct pair_of<__half> { using type = __half2; };
template <> struct pair_of<__nv_bfloat16> { using type = __nv_bfloat162; };

__device__ __forceinline__ float2 unpack2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 unpack2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
__device__ __forceinline__ __half2 pack2(float a, float b, __half2) { return __floats2half2_rn(a, b); }
__device__ __forceinline__ __nv_bfloat162 pack2(float a, float b, __nv_bfloat162) { return __floats2bfloat162_rn(a, b); }

// qkv [B, T, H + 2*KV, hd]; pos int64 [T]; cos / sin f32 [max_seq, hd/2] (rotate-half convention:
// element i pairs with element i + hd/2); q_out [B, H, T, hd]; k_cache / v_cache [B, KV, max_seq, hd].
// One thread handles two neighbouring i (a 32-bit pair) of both halves of one head.
template <typename T>
__global__ void __launch_bounds__(256) rope_kv_kernel(const T* qkv, const long long* pos,
                                                      const float* cosv, const float* sinv,
                                                      T* q_out, T* k_cache, T* v_cache,
                                                      int B, int Tn, int H, int KV, int hd, int max_seq) {
    using P = typename pair_of<T>::type;
    pdl_launch_dependents();
    pdl_wait();
    const int half = hd / 2, pairs = half / 2, heads = H + 2 * KV;
    const long long total = static_cast<long long>(B) * Tn * heads * pairs;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int ip = static_cast<int>(idx % pairs);
        const int h = static_cast<int>((idx / pairs) % heads);
        const int t = static_cast<int>((idx / (static_cast<long long>(pairs) * heads)) % Tn);
        const int b = static_cast<int>(idx / (static_cast<long long>(pairs) * heads * Tn));
        const long long p = pos[t];
        // A position outside the cache would index the cos / sin tables and the caches out of
        // bounds: such a token is skipped (nothing read at p, nothing stored) and reported in the
        // device status word, since the position is a device value the host never sees.
        if (p < 0 || p >= max_seq) {
            if (ip == 0 && h == 0) atomicOr(&g_status, STATUS_GLUE_POS);
            continue;
        }
        const T* src = qkv + ((static_cast<size_t>(b) * Tn + t) * heads + h) * hd;
        const float2 x1 = unpack2(*reinterpret_cast<const P*>(src + 2 * ip));
        const float2 x2 = unpack2(*reinterpret_cast<const P*>(src + half + 2 * ip));
        T* dst;
        float2 o1 = x1, o2 = x2;
        if (h < H + KV) {                                      // Q and K heads are rotated
            const float2 c = *reinterpret_cast<const float2*>(cosv + p * half + 2 * ip);
            const float2 s = *reinterpret_cast<const float2*>(sinv + p * half + 2 * ip);
            o1 = make_float2(x1.x * c.x - x2.x * s.x, x1.y * c.y - x2.y * s.y);
            o2 = make_float2(x2.x * c.x + x1.x * s.x, x2.y * c.y + x1.y * s.y);
        }
        if (h < H) dst = q_out + ((static_cast<size_t>(b) * H + h) * Tn + t) * hd;
        else if (h < H + KV) dst = k_cache + ((static_cast<size_t>(b) * KV + (h - H)) * max_seq + p) * hd;
        else dst = v_cache + ((static_cast<size_t>(b) * KV + (h - H - KV)) * max_seq + p) * hd;
        *reinterpret_cast<P*>(dst + 2 * ip) = pack2(o1.x, o1.y, P());
        *reinterpret_cast<P*>(dst + half + 2 * ip) = pack2(o2.x, o2.y, P());
    }
}

// The same step for an FP8 KV cache: K (rotated) and V are rounded to the activation type, as the
// 16-bit cache would hold them, and then quantized per token and KV head exactly as
// quantize_weight quantizes a row (tfp8/quantize.py:15-36 of the reference: power-of-two scale
// 2^ceil(log2(amax / fmax)), 1 for an all-zero row, round to nearest even, saturating): codes
// k_codes / v_codes u8 [B, KV, max_seq, hd] and one FP32 scale per (sequence, KV head, position).
// One warp per (sequence, token, head); hd = 128: lane l holds elements 2l, 2l + 1 of both halves.
template <typename T, int FMT>
__global__ void __launch_bounds__(256) rope_kv_fp8_kernel(const T* qkv, const long long* pos,
                                                          const float* cosv, const float* sinv,
                                                          T* q_out, uint8_t* k_codes,
                                                          float* k_scale, uint8_t* v_codes,
                                                          float* v_scale, int B, int Tn, int H, int KV, int max_seq) {
    using P = typename pair_of<T>::type;
    pdl_launch_dependents();
    pdl_wait();
    constexpr int hd = 128, half = 64;
    constexpr float fmax = FMT == TFP8B_E4M3FN ? 448.f : 57344.f;
    const int heads = H + 2 * KV, lane = threadIdx.x & 31;
    const long long total = static_cast<long long>(B) * Tn * heads;
    const long long w0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long wstep = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long idx = w0; idx < total; idx += wstep) {
        const int h = static_cast<int>(idx % heads);
        const int t = static_cast<int>((idx / heads) % Tn);
        const int b = static_cast<int>(idx / (static_cast<long long>(heads) * Tn));
        const long long p = pos[t];
        if (p < 0 || p >= max_seq) {                           // outside the cache: skipped and reported
            if (lane == 0 && h == 0) atomicOr(&g_status, STATUS_GLUE_POS);
            continue;
        }
        const T* src = qkv + ((static_cast<size_t>(b) * Tn + t) * heads + h) * hd;
        const float2 x1 = unpack2(*reinterpret_cast<const P*>(src + 2 * lane));
        const float2 x2 = unpack2(*reinterpret_cast<const P*>(src + half + 2 * lane));
        float2 o1 = x1, o2 = x2;
        if (h < H + KV) {                                      // Q and K heads are rotated
            const float2 c = *reinterpret_cast<const float2*>(cosv + p * half + 2 * lane);
            const float2 sn = *reinterpret_cast<const float2*>(sinv + p * half + 2 * lane);
            o1 = make_float2(x1.x * c.x - x2.x * sn.x, x1.y * c.y - x2.y * sn.y);
            o2 = make_float2(x2.x * c.x + x1.x * sn.x, x2.y * c.y + x1.y * sn.y);
        }
        const P r1 = pack2(o1.x, o1.y, P()), r2 = pack2(o2.x, o2.y, P());
        if (h < H) {
            T* dst = q_out + ((static_cast<size_t>(b) * H + h) * Tn + t) * hd;
            *reinterpret_cast<P*>(dst + 2 * lane) = r1;
            *reinterpret_cast<P*>(dst + half + 2 * lane) = r2;
            continue;
        }
        const bool is_k = h < H + KV;
        const size_t row = (static_cast<size_t>(b) * KV + (is_k ? h - H : h - H - KV)) * max_seq + p;
        const float2 a = unpack2(r1), c2 = unpack2(r2);
        float v[4] = {a.x, a.y, c2.x, c2.y};
        float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const float sc = scale_from_amax(m, fmax, 1);
        const uint32_t sb = __float_as_uint(sc);
        if (sb >= 0x00800000u && sb <= 0x7E800000u) {          // a power of two by construction: its reciprocal is exact
            const float inv = __uint_as_float(0x7F000000u - sb);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] *= inv;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = __fdiv_rn(v[i], sc);
        }
        uint32_t c01 = enc2_hw<FMT>(v[0], v[1]), c23 = enc2_hw<FMT>(v[2], v[3]);
        constexpr uint32_t NAN_PROBE = FMT == TFP8B_E4M3FN ? 0x0101u : 0x0404u;
        if (((c01 & 0x7F7Fu) + NAN_PROBE) & 0x8080u) c01 = encode1<FMT>(v[0], TFP8B_NAN_CAST) | (encode1<FMT>(v[1], TFP8B_NAN_CAST) << 8);
        if (((c23 & 0x7F7Fu) + NAN_PROBE) & 0x8080u) c23 = encode1<FMT>(v[2], TFP8B_NAN_CAST) | (encode1<FMT>(v[3], TFP8B_NAN_CAST) << 8);
        uint8_t* dst = (is_k ? k_codes : v_codes) + row * hd;
        *reinterpret_cast<uint16_t*>(dst + 2 * lane) = static_cast<uint16_t>(c01);
        *reinterpret_cast<uint16_t*>(dst + half + 2 * lane) = static_cast<uint16_t>(c23);
        if (lane == 0) (is_k ? k_scale : v_scale)[row] = sc;
    }
}

// gu [rows, 2F] -> out [rows, F] = silu(gu[:, :F]) * gu[:, F:]; eight elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* gu, T* out, long long rows, int F) {
    using P = typename pair_of<T>::type;
    pdl_launch_dependents();
    pdl_wait();
    const int vec = F / 8;
    const long long total = rows * vec;
    for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = idx / vec;
        const int c = static_cast<int>(idx % vec) * 8;
        const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c);
        const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
        uint4 o;
        const P* gp = reinterpret_cast<const P*>(&g);
        const P* up = reinterpret_cast<const P*>(&u);
        P* op = reinterpret_cast<P*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = unpack2(gp[i]), b = unpack2(up[i]);
            op[i] = pack2(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y, P());
        }
        *reinterpret_cast<uint4*>(out + r * F + c) = o;
    }
}

// x[r, :] += delta[r, :] (rounded to T, stored), out[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * w.
// One CTA per row, eight elements per thread and step, the row kept in registers between the two
// passes when it fits (dim <= 8 * 256 * ADD_NORM_KEEP).
constexpr int ADD_NORM_THREADS = 256;
constexpr int ADD_NORM_KEEP = 4;
template <typename T>
__global__ void __launch_bounds__(ADD_NORM_THREADS) add_rmsnorm_kernel(T* x, const T* delta,
                                                                       const T* w, T* out,
                                                                       int dim, float eps) {
    using P = typename pair_of<T>::type;
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = static_cast<size_t>(blockIdx.x) * dim;
    const int nvec = dim / 8;
    uint4 keep[ADD_NORM_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ADD_NORM_KEEP; ++it) {
        const int v = threadIdx.x + it * ADD_NORM_THREADS;
        if (v < nvec) {
            uint4 a = *reinterpret_cast<const uint4*>(x + row + v * 8);
            if (delta) {
                const uint4 d = *reinterpret_cast<const uint4*>(delta + row + v * 8);
                P* ap = reinterpret_cast<P*>(&a);
                const P* dp = reinterpret_cast<const P*>(&d);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = unpack2(ap[i]), g = unpack2(dp[i]);
                    ap[i] = pack2(f.x + g.x, f.y + g.y, P());
                }
                *reinterpret_cast<uint4*>(x + row + v * 8) = a;
            }
            keep[it] = a;
            const P* ap = reinterpret_cast<const P*>(&a);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = unpack2(ap[i]); ss += f.x * f.x + f.y * f.y; }
        }
    }
    for (int v = threadIdx.x + ADD_NORM_KEEP * ADD_NORM_THREADS; v < nvec; v += ADD_NORM_THREADS) {   // long rows: the tail
        uint4 a = *reinterpret_cast<const uint4*>(x + row + v * 8);
        P* ap = reinterpret_cast<P*>(&a);
        if (delta) {
            const uint4 d = *reinterpret_cast<const uint4*>(delta + row + v * 8);
            const P* dp = reinterpret_cast<const P*>(&d);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = unpack2(ap[i]), g = unpack2(dp[i]); ap[i] = pack2(f.x + g.x, f.y + g.y, P()); }
            *reinterpret_cast<uint4*>(x + row + v * 8) = a;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = unpack2(ap[i]); ss += f.x * f.x + f.y * f.y; }
    }
    __shared__ float s_part[ADD_NORM_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < ADD_NORM_THREADS / 32; ++i) ss += s_part[i];
    const float rstd = rsqrtf(ss / static_cast<float>(dim) + eps);
    auto emit = [&](int v, const uint4& a) {
        const uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
        const P* ap = reinterpret_cast<const P*>(&a);
        const P* wp = reinterpret_cast<const P*>(&wv);
        uint4 o;
        P* op = reinterpret_cast<P*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = unpack2(ap[i]), g = unpack2(wp[i]);
            op[i] = pack2(f.x * rstd * g.x, f.y * rstd * g.y, P());
        }
        *reinterpret_cast<uint4*>(out + row + v * 8) = o;
    };
#pragma unroll
    for (int it = 0; it < ADD_NORM_KEEP; ++it) {
        const int v = threadIdx.x + it * ADD_NORM_THREADS;
        if (v < nvec) emit(v, keep[it]);
    }
    for (int v = threadIdx.x + ADD_NORM_KEEP * ADD_NORM_THREADS; v < nvec; v += ADD_NORM_THREADS)
        emit(v, *reinterpret_cast<const uint4*>(x + row + v * 8));       // re-read what this thread stored
}

// ------------------------------------------------------------------ all-reduce + residual + RMSNorm
// Tensor-parallel decode: after a row-parallel projection every rank holds an FP32 partial
// [rows, dim] of the same output. A NCCL all-reduce of those 8-32 KB costs ~19 us inside a decode
// step, 64 times per token; this kernel does the exchange itself, one CTA per row:
//   1. push this rank's partial row into every peer's receive slot (peer-mapped memory, plain
//      16-byte stores over NVLink), fence, then write the call's sequence number into the peer's
//      flag for (this rank, row);
//   2. wait (bounded) until every peer's flag for this row shows the same sequence number;
//   3. add the partials in rank order (every rank computes bit-identical sums), round to the
//      activation type, add to the residual, RMSNorm.
// Receive slots and flags are double-buffered by the parity of the sequence number: a rank can
// run at most one call ahead of a peer (it needs the peer's flag of call k to finish call k), so
// the slot it overwrites in call k + 2 has been read. The sequence number lives in device memory
// and is advanced by the last CTA of each call, which is what makes the kernel replayable from a
// CUDA graph. Every rank must issue the same calls in the same order.
struct ArParams {
    float* recv[8];            // recv[r]: rank r's receive area [2][world][max_rows][dim] (recv[rank] is local)
    unsigned int* flag[8];     // flag[r]: rank r's flags [2][world][max_rows]
    unsigned int* state;       // local: {sequence number of the last finished call, CTAs done in the running call}
    int rank, world, max_rows;
    long long wait_cycles;     // SM clock cycles a CTA waits for a peer's flag before it gives up
};
constexpr int AR_THREADS = 256;
template <typename T>
__global__ void __launch_bounds__(AR_THREADS) allreduce_add_rmsnorm_kernel(T* x, const float* part,
                                                                           const T* w, T* out,
                                                                           int dim, float eps, const ArParams ar) {
    using P = typename pair_of<T>::type;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, nvec = dim / 4;
    const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(ar.state) + 1u;
    const size_t slot_elems = static_cast<size_t>(ar.max_rows) * dim;
    const size_t buf_off = static_cast<size_t>(seq & 1u) * ar.world * slot_elems;
    const size_t flag_off = static_cast<size_t>(seq & 1u) * ar.world * ar.max_rows;
    const float* mine = part + static_cast<size_t>(row) * dim;
    __shared__ int s_gave_up;
    if (threadIdx.x == 0) s_gave_up = 0;
    // 1. push
    for (int v = threadIdx.x; v < nvec; v += AR_THREADS) {
        const float4 a = reinterpret_cast<const float4*>(mine)[v];
        for (int r = 0; r < ar.world; ++r)
            if (r != ar.rank)
                reinterpret_cast<float4*>(ar.recv[r] + buf_off + ar.rank * slot_elems + static_cast<size_t>(row) * dim)[v] = a;
    }
    __threadfence_system();
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < ar.world && static_cast<int>(threadIdx.x) != ar.rank) {
        unsigned int* f = ar.flag[threadIdx.x] + flag_off + ar.rank * ar.max_rows + row;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
        // 2. wait for the same peer's row
        const unsigned int* g = ar.flag[ar.rank] + flag_off + threadIdx.x * ar.max_rows + row;
        const long long t0 = clock64();
        unsigned int got;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(g) : "memory");
            if (got == seq) break;
            if (clock64() - t0 > ar.wait_cycles) { atomicOr(&g_status, STATUS_GLUE_WAIT); s_gave_up = 1; break; }
            __nanosleep(100);
        }
    }
    __syncthreads();
    // A peer that never answered: its slot holds stale data, so a sum would be silently wrong while
    // the peer (which did receive this rank's partial) computes the right one. The row is poisoned
    // instead -- NaN in the residual and in the output -- so the failure shows in every later token,
    // and the status word says why.
    const bool gave_up = s_gave_up != 0;
    // 3. sum in rank order, residual, norm (rows of up to 4 * AR_THREADS * AR_KEEP floats stay in registers)
    constexpr int AR_KEEP = 4;
    float4 keep[AR_KEEP];
    float ss = 0.f;
    const size_t xrow = static_cast<size_t>(row) * dim;
    const float* local = ar.recv[ar.rank] + buf_off + static_cast<size_t>(row) * dim;
#pragma unroll
    for (int it = 0; it < AR_KEEP; ++it) {
        const int v = threadIdx.x + it * AR_THREADS;
        if (v < nvec) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < ar.world; ++r) {
                const float4 a = r == ar.rank ? reinterpret_cast<const float4*>(mine)[v]
                                              : __ldcg(reinterpret_cast<const float4*>(local + r * slot_elems) + v);
                t.x += a.x; t.y += a.y; t.z += a.z; t.w += a.w;
            }
            if (gave_up) t.x = t.y = t.z = t.w = __int_as_float(0x7FC00000);
            const uint2 xr = *reinterpret_cast<const uint2*>(x + xrow + v * 4);
            const P* xp = reinterpret_cast<const P*>(&xr);
            // the reduced projection output is rounded to the activation type, then added (as the
            // unfused sequence all-reduce -> cast -> add does)
            const float2 d01 = unpack2(pack2(t.x, t.y, P())), d23 = unpack2(pack2(t.z, t.w, P()));
            const float2 x01 = unpack2(xp[0]), x23 = unpack2(xp[1]);
            uint2 xo;
            P* op = reinterpret_cast<P*>(&xo);
            op[0] = pack2(x01.x + d01.x, x01.y + d01.y, P());
            op[1] = pack2(x23.x + d23.x, x23.y + d23.y, P());
            *reinterpret_cast<uint2*>(x + xrow + v * 4) = xo;
            const float2 n01 = unpack2(op[0]), n23 = unpack2(op[1]);
            keep[it] = make_float4(n01.x, n01.y, n23.x, n23.y);
            ss += n01.x * n01.x + n01.y * n01.y + n23.x * n23.x + n23.y * n23.y;
        }
    }
    __shared__ float s_part[AR_THREADS / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int i = 0; i < AR_THREADS / 32; ++i) ss += s_part[i];
    const float rstd = rsqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
    for (int it = 0; it < AR_KEEP; ++it) {
        const int v = threadIdx.x + it * AR_THREADS;
        if (v < nvec) {
            const uint2 wr = *reinterpret_cast<const uint2*>(w + v * 4);
            const P* wp = reinterpret_cast<const P*>(&wr);
            const float2 w01 = unpack2(wp[0]), w23 = unpack2(wp[1]);
            uint2 o;
            P* op = reinterpret_cast<P*>(&o);
            op[0] = pack2(keep[it].x * rstd * w01.x, keep[it].y * rstd * w01.y, P());
            op[1] = pack2(keep[it].z * rstd * w23.x, keep[it].w * rstd * w23.y, P());
            *reinterpret_cast<uint2*>(out + xrow + v * 4) = o;
        }
    }
    // the last CTA of the call advances the sequence number
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(ar.state + 1, 1u) == gridDim.x - 1) {
            ar.state[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(ar.state) = seq;
        }
    }
}

// out[r] = index of the largest logits[r, :]; the lowest index among equals; a NaN counts as the
// largest value (the first NaN wins), as torch.argmax does. One CTA per row.
constexpr int ARGMAX_THREADS = 1024;
__device__ __forceinline__ bool argmax_better(float v, long long i, float bv, long long bi) {
    const bool vn = v != v, bn = bv != bv;
    if (vn || bn) return vn && (!bn || i < bi);
    return v > bv || (v == bv && i < bi);
}
template <typename T>
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const T* logits, long long* out,
                                                                long long n, long long row_pitch) {
    using P = typename pair_of<T>::type;
    pdl_launch_dependents();
    pdl_wait();
    const T* row = logits + static_cast<size_t>(blockIdx.x) * row_pitch;
    float best = -INFINITY;
    long long bi = 0x7fffffffffffffffll;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const long long nvec = vec_ok ? n / 8 : 0;
    for (long long v = threadIdx.x; v < nvec; v += ARGMAX_THREADS) {
        const uint4 a = *reinterpret_cast<const uint4*>(row + v * 8);
        const P* ap = reinterpret_cast<const P*>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = unpack2(ap[i]);
            if (argmax_better(f.x, v * 8 + 2 * i, best, bi)) { best = f.x; bi = v * 8 + 2 * i; }
            if (argmax_better(f.y, v * 8 + 2 * i + 1, best, bi)) { best = f.y; bi = v * 8 + 2 * i + 1; }
        }
    }
    for (long long i = nvec * 8 + threadIdx.x; i < n; i += ARGMAX_THREADS) {
        const float f = to_f32(row[i]);
        if (argmax_better(f, i, best, bi)) { best = f; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
    }
    __shared__ float s_v[ARGMAX_THREADS / 32];
    __shared__ long long s_i[ARGMAX_THREADS / 32];
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = best; s_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = s_v[threadIdx.x]; bi = s_i[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (argmax_better(ov, oi, best, bi)) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = bi;
    }
}

// ------------------------------------------------------------------ decode attention
// One query token per sequence against cache positions [0, pos]: out[b, h, :] = softmax(q . K^T
// / sqrt(hd)) V. The KV range of one (sequence, KV head) is split into chunks of at most 64
// positions, one CTA each, so that a batch-1 step still fills the machine; a CTA serves up to
// four of the query heads that share its KV head, and writes an unnormalised partial (running
// maximum, sum, weighted V) that attn_merge_kernel combines. Every global load of a phase is
// issued before its first use (the chunk is short: one memory round trip per phase). FP32
// arithmetic throughout. hd = 128.
#ifndef TFP8B_ATT_THREADS
#define TFP8B_ATT_THREADS 128
#endif
constexpr int ATT_THREADS = TFP8B_ATT_THREADS;
constexpr int ATT_HD = 128;
constexpr int ATT_G = 4;             // query heads per CTA (a KV head with more is served by several CTAs)
constexpr int ATT_CHUNK = 64;        // positions per CTA at most
constexpr int ATT_PW = ATT_CHUNK / (ATT_THREADS / 32);      // positions per warp: 16
template <typename T>
__global__ void __launch_bounds__(ATT_THREADS) attn_partial_kernel(const T* q, const T* kc,
                                                                   const T* vc, const long long* pos,
                                                                   float* part, int H, int KV, int S, int nsplit,
                                                                   float scale_log2e, int early) {
    using P = typename pair_of<T>::type;
    if (early) pdl_launch_dependents();
    pdl_wait();
    const int G = H / KV, ngrp = (G + ATT_G - 1) / ATT_G;
    int id = blockIdx.x;
    const int split = id % nsplit; id /= nsplit;
    const int grp = id % ngrp; id /= ngrp;
    const int kvh = id % KV, b = id / KV;
    const int h0 = kvh * G + grp * ATT_G, nh = min(ATT_G, G - grp * ATT_G);      // this CTA's query heads
    const int len = static_cast<int>(min(static_cast<long long>(S), pos[0] + 1));
    const int chunk = min(ATT_CHUNK, (len + nsplit - 1) / nsplit);
    const int s0 = split * chunk, n = max(0, min(len, s0 + chunk) - s0);
    __shared__ float s_sc[ATT_G][ATT_CHUNK];
    __shared__ float s_m[ATT_G], s_l[ATT_G];
    __shared__ __align__(16) float s_acc[ATT_THREADS / 32][ATT_G][ATT_HD];     // written as float4
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* kbase = kc + ((static_cast<size_t>(b) * KV + kvh) * S + s0) * ATT_HD;
    const T* vbase = vc + ((static_cast<size_t>(b) * KV + kvh) * S + s0) * ATT_HD;
    // ---- scores: warp w takes positions [16 w, 16 w + 16); 8 lanes per position, 16 dims per lane
    {
        const int sub = lane & 7, slot = lane >> 3;
        uint4 kr[ATT_PW / 4][2];
#pragma unroll
        for (int it = 0; it < ATT_PW / 4; ++it) {
            const int j = warp * ATT_PW + it * 4 + slot;
            if (j < n) {
                const uint4* kp = reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(j) * ATT_HD + sub * 16);
                kr[it][0] = kp[0]; kr[it][1] = kp[1];
            } else {
                kr[it][0] = kr[it][1] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        float qf[ATT_G][16];
#pragma unroll
        for (int g = 0; g < ATT_G; ++g) {
            const T* qp = q + (static_cast<size_t>(b) * H + h0 + min(g, nh - 1)) * ATT_HD + sub * 16;
            const uint4 a0 = reinterpret_cast<const uint4*>(qp)[0], a1 = reinterpret_cast<const uint4*>(qp)[1];
            const P* p0 = reinterpret_cast<const P*>(&a0);
            const P* p1 = reinterpret_cast<const P*>(&a1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f0 = unpack2(p0[i]), f1 = unpack2(p1[i]);
                qf[g][2 * i] = f0.x * scale_log2e; qf[g][2 * i + 1] = f0.y * scale_log2e;
                qf[g][8 + 2 * i] = f1.x * scale_log2e; qf[g][9 + 2 * i] = f1.y * scale_log2e;
            }
        }
#pragma unroll
        for (int it = 0; it < ATT_PW / 4; ++it) {
            const int j = warp * ATT_PW + it * 4 + slot;
            float kf[16];
            const P* p0 = reinterpret_cast<const P*>(&kr[it][0]);
            const P* p1 = reinterpret_cast<const P*>(&kr[it][1]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f0 = unpack2(p0[i]), f1 = unpack2(p1[i]);
                kf[2 * i] = f0.x; kf[2 * i + 1] = f0.y; kf[8 + 2 * i] = f1.x; kf[9 + 2 * i] = f1.y;
            }
#pragma unroll
            for (int g = 0; g < ATT_G; ++g) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) d = fmaf(qf[g][i], kf[i], d);
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                if (sub == 0 && j < n) s_sc[g][j] = d;
            }
        }
    }
    // ---- the V rows of this warp's positions, requested now, used after the softmax
    uint2 vr[ATT_PW];                                  // lane owns dims 4 lane .. 4 lane + 3
#pragma unroll
    for (int it = 0; it < ATT_PW; ++it) {
        const int j = warp * ATT_PW + it;
        vr[it] = j < n ? *reinterpret_cast<const uint2*>(vbase + static_cast<size_t>(j) * ATT_HD + lane * 4) : make_uint2(0u, 0u);
    }
    __syncthreads();
    // ---- per head: maximum, exponentials, sum (warp g serves head g)
    if (warp < nh) {
        const int g = warp;
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, s_sc[g][j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int j = lane; j < n; j += 32) {
            const float e = exp2f(s_sc[g][j] - m);
            s_sc[g][j] = e;
            l += e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) { s_m[g] = m; s_l[g] = l; }
    }
    __syncthreads();
    // ---- weighted V over this warp's positions, then the four warps' sums are added
    float acc[ATT_G][4];
#pragma unroll
    for (int g = 0; g < ATT_G; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;
#pragma unroll
    for (int it = 0; it < ATT_PW; ++it) {
        const int j = warp * ATT_PW + it;
        if (j < n) {
            const P* vp = reinterpret_cast<const P*>(&vr[it]);
            const float2 v01 = unpack2(vp[0]), v23 = unpack2(vp[1]);
#pragma unroll
            for (int g = 0; g < ATT_G; ++g) {
                const float w = s_sc[g][j];
                acc[g][0] = fmaf(w, v01.x, acc[g][0]); acc[g][1] = fmaf(w, v01.y, acc[g][1]);
                acc[g][2] = fmaf(w, v23.x, acc[g][2]); acc[g][3] = fmaf(w, v23.y, acc[g][3]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < ATT_G; ++g)
        *reinterpret_cast<float4*>(&s_acc[warp][g][lane * 4]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    __syncthreads();
    // partial record per (b, head, split): [m, l, acc[128]]
    for (int g = 0; g < nh; ++g) {
        float* rec = part + ((static_cast<size_t>(b) * H + h0 + g) * nsplit + split) * (ATT_HD + 2);
        if (threadIdx.x < ATT_HD) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_THREADS / 32; ++w) sum += s_acc[w][g][threadIdx.x];
            rec[2 + threadIdx.x] = sum;
        }
        if (threadIdx.x == 0) { rec[0] = n > 0 ? s_m[g] : -INFINITY; rec[1] = n > 0 ? s_l[g] : 0.f; }
    }
    if (!early) pdl_launch_dependents();
}

// Decode attention over an FP8 KV cache (codes u8 [B, KV, S, 128], one FP32 scale per position),
// both products on the tensor cores (mma.sync m16n8k16, fp16 operands, FP32 accumulate): with
// scalar FP32 arithmetic the kernel issued 0.25 warp instructions per byte of cache, more than an
// SM can issue in the time its share of HBM delivers that byte, and reading half the bytes of a
// 16-bit cache bought nothing.
//   scores^T [16 positions x 8 heads] = K [16 x 128] Q^T: A = codes decoded to fp16 (exact), one
//     position per fragment row; B = Q, the KV head's query heads as columns (4 of 8 used). The
//     128 dims are contracted in an order that lets a lane read its codes as two 16-byte loads:
//     lane (g, t) holds bytes [32 t, 32 t + 32) of rows g and g + 8, and k-step c of 8 contracts
//     dims 32 t + 4 c .. + 3; Q is loaded in the same order. The K scale and 1 / sqrt(hd) are
//     applied to the FP32 scores.
//   out^T [128 dims x 8 heads] = V^T [128 x 16 positions] P^T: the contraction now runs over
//     positions, which is the slow index of the cache; a fragment register wants the same dim of
//     two neighbouring positions, and a byte permute of the two positions' code words makes that
//     pair before the conversion. P = exp2(score - max) is rounded to fp16 as a high and a low
//     part (two MMAs), the V scale relative to the chunk's largest rides on the decoded V (a power
//     of two: exact), the largest itself on the FP32 result.
// A CTA serves one (sequence, KV head, up to four query heads, 128 or 256 positions); a warp 32 of them.
constexpr int ATT8_PW = 32;                                    // positions per warp: two 16-position blocks

__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t to_f16x2(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ uint32_t to_f16x2(__nv_bfloat162 v) {      // every bf16 in fp16's range is exact in fp16
    const float2 f = __bfloat1622float2(v);
    __half2 h = __floats2half2_rn(f.x, f.y);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T, int FMT, int NW>
__global__ void __launch_bounds__(32 * NW) attn_partial_fp8_kernel(const T* q, const uint8_t* kc, const float* ksc, const uint8_t* vc,
                                                                       const float* vsc, const long long* pos, float* part, int H, int KV,
                                                                       int S, int nsplit, float scale_log2e, int early) {
    using P = typename pair_of<T>::type;
    constexpr int ATT8_CHUNK = ATT8_PW * NW;                       // positions per CTA: 128 (four warps) or 256 (eight)
    if (early) pdl_launch_dependents();
    pdl_wait();
    const int G = H / KV, ngrp = (G + ATT_G - 1) / ATT_G;
    int id = blockIdx.x;
    const int split = id % nsplit; id /= nsplit;
    const int grp = id % ngrp; id /= ngrp;
    const int kvh = id % KV, b = id / KV;
    const int h0 = kvh * G + grp * ATT_G, nh = min(ATT_G, G - grp * ATT_G);
    const int len = static_cast<int>(min(static_cast<long long>(S), pos[0] + 1));
    const int chunk = min(ATT8_CHUNK, (len + nsplit - 1) / nsplit);
    const int s0 = split * chunk, n = max(0, min(len, s0 + chunk) - s0);
    __shared__ __align__(16) float s_sc[ATT_G][ATT8_CHUNK];         // scores
    __shared__ __align__(16) __half s_ph[ATT_G][ATT8_CHUNK];        // softmax weights, high part (read as pairs)
    __shared__ __align__(16) __half s_pl[ATT_G][ATT8_CHUNK];        // ... and low part
    __shared__ float s_m[ATT_G], s_l[ATT_G], s_vmax;
    __shared__ __align__(16) float s_acc[NW][ATT_G][ATT_HD];   // written as pairs of floats
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const size_t row0 = (static_cast<size_t>(b) * KV + kvh) * S + s0;
    const uint8_t* kbase = kc + row0 * ATT_HD;
    const uint8_t* vbase = vc + row0 * ATT_HD;
    // ---- scores
    {
        // Q of head g (columns 4..7 of the B operand stay zero), dims [32 t, 32 t + 32) as 16 fp16 pairs
        uint32_t qreg[16];
        if (g < nh) {
            const uint4* qp = reinterpret_cast<const uint4*>(q + (static_cast<size_t>(b) * H + h0 + g) * ATT_HD + t * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = qp[i];
                const P* pp = reinterpret_cast<const P*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) qreg[4 * i + e] = to_f16x2(pp[e]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) qreg[i] = 0u;
        }
#pragma unroll
        for (int blk = 0; blk < ATT8_PW / 16; ++blk) {
            const int j0 = warp * ATT8_PW + blk * 16 + g, j1 = j0 + 8;
            uint4 k0[2], k1[2];
            float ks0 = 0.f, ks1 = 0.f;
            if (j0 < n) {
                const uint4* kp = reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(j0) * ATT_HD + t * 32);
                k0[0] = __ldcg(kp); k0[1] = __ldcg(kp + 1);
                ks0 = __ldcg(ksc + row0 + j0) * scale_log2e;
            } else {
                k0[0] = k0[1] = make_uint4(0u, 0u, 0u, 0u);
            }
            if (j1 < n) {
                const uint4* kp = reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(j1) * ATT_HD + t * 32);
                k1[0] = __ldcg(kp); k1[1] = __ldcg(kp + 1);
                ks1 = __ldcg(ksc + row0 + j1) * scale_log2e;
            } else {
                k1[0] = k1[1] = make_uint4(0u, 0u, 0u, 0u);
            }
            const uint32_t w0[8] = {k0[0].x, k0[0].y, k0[0].z, k0[0].w, k0[1].x, k0[1].y, k0[1].z, k0[1].w};
            const uint32_t w1[8] = {k1[0].x, k1[0].y, k1[0].z, k1[0].w, k1[1].x, k1[1].y, k1[1].z, k1[1].w};
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int cstep = 0; cstep < 8; ++cstep) {
                uint32_t a0, a2, a1, a3;
                dec4<FMT, false>(w0[cstep], a0, a2);          // row g: dims +0,+1 | +2,+3
                dec4<FMT, false>(w1[cstep], a1, a3);          // row g + 8
                mma16816(c, a0, a1, a2, a3, qreg[2 * cstep], qreg[2 * cstep + 1]);
            }
            // c0, c1: position j0, heads 2t, 2t + 1; c2, c3: position j1
            if (t < 2) {
                const int hA = 2 * t, hB = 2 * t + 1;
                if (j0 < n) { if (hA < nh) s_sc[hA][j0] = c[0] * ks0; if (hB < nh) s_sc[hB][j0] = c[1] * ks0; }
                if (j1 < n) { if (hA < nh) s_sc[hA][j1] = c[2] * ks1; if (hB < nh) s_sc[hB][j1] = c[3] * ks1; }
            }
        }
    }
    // ---- the V codes and scales of this warp's positions, requested now, used after the softmax:
    // lane (g, t) takes dims [16 g, 16 g + 16) of positions 2t, 2t + 1, 2t + 8, 2t + 9 of each block
    uint4 vv[ATT8_PW / 16][4];
    float vsr[ATT8_PW / 16][4];
#pragma unroll
    for (int blk = 0; blk < ATT8_PW / 16; ++blk) {
        const int pb = warp * ATT8_PW + blk * 16;
        const int pj[4] = {pb + 2 * t, pb + 2 * t + 1, pb + 2 * t + 8, pb + 2 * t + 9};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (pj[u] < n) {
                vv[blk][u] = __ldcg(reinterpret_cast<const uint4*>(vbase + static_cast<size_t>(pj[u]) * ATT_HD + g * 16));
                vsr[blk][u] = __ldcg(vsc + row0 + pj[u]);
            } else {
                vv[blk][u] = make_uint4(0u, 0u, 0u, 0u);
                vsr[blk][u] = 0.f;
            }
        }
    }
    __syncthreads();
    // ---- per head: maximum, exponentials (fp16 high + low part), sum; one warp also finds the
    // chunk's largest V scale
    if (warp < nh) {
        const int hh = warp;
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, s_sc[hh][j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int j = lane; j < ATT8_CHUNK; j += 32) {
            float e = 0.f;
            if (j < n) { e = exp2f(s_sc[hh][j] - m); l += e; }
            const __half hi = __float2half_rn(e);
            s_ph[hh][j] = hi;
            s_pl[hh][j] = __float2half_rn(e - __half2float(hi));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) { s_m[hh] = m; s_l[hh] = l; }
    }
    if (warp == NW - 1) {
        float vm = 0.f;
        for (int j = lane; j < n; j += 32) vm = fmaxf(vm, __ldcg(vsc + row0 + j));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, o));
        if (lane == 0) s_vmax = vm > 0.f ? vm : 1.f;
    }
    __syncthreads();
    // ---- out^T = V^T P^T over this warp's positions
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const float inv_vmax = 1.f / s_vmax;                          // a power of two: exact
#pragma unroll
    for (int blk = 0; blk < ATT8_PW / 16; ++blk) {
        const int pb = warp * ATT8_PW + blk * 16;
        // scales relative to the largest: <= 1; below 2^-24 they round to 0 -- such a row is noise beside the largest
        const __half2 sAB = __floats2half2_rn(vsr[blk][0] * inv_vmax, vsr[blk][1] * inv_vmax);
        const __half2 sCD = __floats2half2_rn(vsr[blk][2] * inv_vmax, vsr[blk][3] * inv_vmax);
        // B operand: P of head g at positions (2t, 2t+1) and (2t+8, 2t+9) of the block
        uint32_t bh0 = 0u, bh1 = 0u, bl0 = 0u, bl1 = 0u;
        if (g < nh) {
            bh0 = *reinterpret_cast<const uint32_t*>(&s_ph[g][pb + 2 * t]); bh1 = *reinterpret_cast<const uint32_t*>(&s_ph[g][pb + 2 * t + 8]);
            bl0 = *reinterpret_cast<const uint32_t*>(&s_pl[g][pb + 2 * t]); bl1 = *reinterpret_cast<const uint32_t*>(&s_pl[g][pb + 2 * t + 8]);
        }
        const uint32_t wA[4] = {vv[blk][0].x, vv[blk][0].y, vv[blk][0].z, vv[blk][0].w}, wB[4] = {vv[blk][1].x, vv[blk][1].y, vv[blk][1].z, vv[blk][1].w};
        const uint32_t wC[4] = {vv[blk][2].x, vv[blk][2].y, vv[blk][2].z, vv[blk][2].w}, wD[4] = {vv[blk][3].x, vv[blk][3].y, vv[blk][3].z, vv[blk][3].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // fragment rows g and g + 8 = dims 16 g + 2 i and 16 g + 2 i + 1: bytes (2i) & 3 and + 1 of word i / 2
            const int w = i >> 1;
            const uint32_t selA = (i & 1) ? 0x0062u : 0x0040u, selB = (i & 1) ? 0x0073u : 0x0051u;    // {x.b, y.b} as a 16-bit pair
            uint32_t a0 = dec2_f16<FMT>(__byte_perm(wA[w], wB[w], selA) & 0xFFFFu);
            uint32_t a1 = dec2_f16<FMT>(__byte_perm(wA[w], wB[w], selB) & 0xFFFFu);
            uint32_t a2 = dec2_f16<FMT>(__byte_perm(wC[w], wD[w], selA) & 0xFFFFu);
            uint32_t a3 = dec2_f16<FMT>(__byte_perm(wC[w], wD[w], selB) & 0xFFFFu);
            __half2 x0 = __hmul2(*reinterpret_cast<__half2*>(&a0), sAB), x1 = __hmul2(*reinterpret_cast<__half2*>(&a1), sAB);
            __half2 x2 = __hmul2(*reinterpret_cast<__half2*>(&a2), sCD), x3 = __hmul2(*reinterpret_cast<__half2*>(&a3), sCD);
            a0 = *reinterpret_cast<uint32_t*>(&x0); a1 = *reinterpret_cast<uint32_t*>(&x1);
            a2 = *reinterpret_cast<uint32_t*>(&x2); a3 = *reinterpret_cast<uint32_t*>(&x3);
            mma16816(o[i], a0, a1, a2, a3, bh0, bh1);
            mma16816(o[i], a0, a1, a2, a3, bl0, bl1);
        }
    }
    // o[i][0], [1]: dim 16 g + 2 i, heads 2t, 2t + 1; o[i][2], [3]: dim 16 g + 2 i + 1
    if (t < 2) {
        const float vmax = s_vmax;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = 16 * g + 2 * i;
            *reinterpret_cast<float2*>(&s_acc[warp][2 * t][d]) = make_float2(o[i][0] * vmax, o[i][2] * vmax);
            *reinterpret_cast<float2*>(&s_acc[warp][2 * t + 1][d]) = make_float2(o[i][1] * vmax, o[i][3] * vmax);
        }
    }
    __syncthreads();
    for (int hh = 0; hh < nh; ++hh) {
        float* rec = part + ((static_cast<size_t>(b) * H + h0 + hh) * nsplit + split) * (ATT_HD + 2);
        if (threadIdx.x < ATT_HD) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) sum += s_acc[w][hh][threadIdx.x];
            rec[2 + threadIdx.x] = sum;
        }
        if (threadIdx.x == 0) { rec[0] = n > 0 ? s_m[hh] : -INFINITY; rec[1] = n > 0 ? s_l[hh] : 0.f; }
    }
    if (!early) pdl_launch_dependents();
}

// The same formulation over a 16-bit (fp16) cache: the K rows are MMA fragments as they are loaded,
// the V pairs of neighbouring positions are made by a permute of 16-bit halves; no scales. A lane
// holds 32 dims of a row as four 16-byte loads (scores) and 16 dims of four positions (output).
template <int NW>
__global__ void __launch_bounds__(32 * NW) attn_partial_f16tc_kernel(const __half* q, const __half* kc, const __half* vc,
                                                                     const long long* pos, float* part, int H, int KV, int S, int nsplit,
                                                                     float scale_log2e, int early) {
    constexpr int CHUNK = ATT8_PW * NW;
    if (early) pdl_launch_dependents();
    pdl_wait();
    const int G = H / KV, ngrp = (G + ATT_G - 1) / ATT_G;
    int id = blockIdx.x;
    const int split = id % nsplit; id /= nsplit;
    const int grp = id % ngrp; id /= ngrp;
    const int kvh = id % KV, b = id / KV;
    const int h0 = kvh * G + grp * ATT_G, nh = min(ATT_G, G - grp * ATT_G);
    const int len = static_cast<int>(min(static_cast<long long>(S), pos[0] + 1));
    const int chunk = min(CHUNK, (len + nsplit - 1) / nsplit);
    const int s0 = split * chunk, n = max(0, min(len, s0 + chunk) - s0);
    __shared__ __align__(16) float s_sc[ATT_G][CHUNK];
    __shared__ __align__(16) __half s_ph[ATT_G][CHUNK];
    __shared__ __align__(16) __half s_pl[ATT_G][CHUNK];
    __shared__ float s_m[ATT_G], s_l[ATT_G];
    __shared__ __align__(16) float s_acc[NW][ATT_G][ATT_HD];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const size_t row0 = (static_cast<size_t>(b) * KV + kvh) * S + s0;
    const __half* kbase = kc + row0 * ATT_HD;
    const __half* vbase = vc + row0 * ATT_HD;
    // ---- scores: lane (g, t) holds dims [32 t, 32 t + 32) of rows g and g + 8; k-step c contracts dims 32 t + 4 c .. + 3
    {
        uint32_t qreg[16];
        if (g < nh) {
            const uint4* qp = reinterpret_cast<const uint4*>(q + (static_cast<size_t>(b) * H + h0 + g) * ATT_HD + t * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = qp[i];
                qreg[4 * i] = v.x; qreg[4 * i + 1] = v.y; qreg[4 * i + 2] = v.z; qreg[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) qreg[i] = 0u;
        }
#pragma unroll
        for (int blk = 0; blk < ATT8_PW / 16; ++blk) {
            const int j0 = warp * ATT8_PW + blk * 16 + g, j1 = j0 + 8;
            uint4 k0[4], k1[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                k0[i] = j0 < n ? __ldcg(reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(j0) * ATT_HD + t * 32) + i) : make_uint4(0u, 0u, 0u, 0u);
                k1[i] = j1 < n ? __ldcg(reinterpret_cast<const uint4*>(kbase + static_cast<size_t>(j1) * ATT_HD + t * 32) + i) : make_uint4(0u, 0u, 0u, 0u);
            }
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 4; ++i) {                       // two k-steps per 16-byte piece
                mma16816(c, k0[i].x, k1[i].x, k0[i].y, k1[i].y, qreg[4 * i], qreg[4 * i + 1]);
                mma16816(c, k0[i].z, k1[i].z, k0[i].w, k1[i].w, qreg[4 * i + 2], qreg[4 * i + 3]);
            }
            if (t < 2) {
                const int hA = 2 * t, hB = 2 * t + 1;
                if (j0 < n) { if (hA < nh) s_sc[hA][j0] = c[0] * scale_log2e; if (hB < nh) s_sc[hB][j0] = c[1] * scale_log2e; }
                if (j1 < n) { if (hA < nh) s_sc[hA][j1] = c[2] * scale_log2e; if (hB < nh) s_sc[hB][j1] = c[3] * scale_log2e; }
            }
        }
    }
    // ---- the V rows of the warp's first block, requested now, used after the softmax (the second
    // block's are requested at the start of the output phase: registers)
    uint4 vv0[4][2];
    {
        const int pb = warp * ATT8_PW;
        const int pj[4] = {pb + 2 * t, pb + 2 * t + 1, pb + 2 * t + 8, pb + 2 * t + 9};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint4* vp = reinterpret_cast<const uint4*>(vbase + static_cast<size_t>(pj[u]) * ATT_HD + g * 16);
            vv0[u][0] = pj[u] < n ? __ldcg(vp) : make_uint4(0u, 0u, 0u, 0u);
            vv0[u][1] = pj[u] < n ? __ldcg(vp + 1) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    __syncthreads();
    // ---- per head: maximum, exponentials (fp16 high + low part), sum
    if (warp < nh) {
        const int hh = warp;
        float m = -INFINITY;
        for (int j = lane; j < n; j += 32) m = fmaxf(m, s_sc[hh][j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int j = lane; j < CHUNK; j += 32) {
            float e = 0.f;
            if (j < n) { e = exp2f(s_sc[hh][j] - m); l += e; }
            const __half hi = __float2half_rn(e);
            s_ph[hh][j] = hi;
            s_pl[hh][j] = __float2half_rn(e - __half2float(hi));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) { s_m[hh] = m; s_l[hh] = l; }
    }
    __syncthreads();
    // ---- out^T = V^T P^T: lane (g, t) takes dims [16 g, 16 g + 16) of positions 2t, 2t + 1, 2t + 8, 2t + 9 of each block
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
    for (int blk = 0; blk < ATT8_PW / 16; ++blk) {
        const int pb = warp * ATT8_PW + blk * 16;
        const int pj[4] = {pb + 2 * t, pb + 2 * t + 1, pb + 2 * t + 8, pb + 2 * t + 9};
        uint4 vv[4][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (blk == 0) {
                vv[u][0] = vv0[u][0]; vv[u][1] = vv0[u][1];
            } else {
                const uint4* vp = reinterpret_cast<const uint4*>(vbase + static_cast<size_t>(pj[u]) * ATT_HD + g * 16);
                vv[u][0] = pj[u] < n ? __ldcg(vp) : make_uint4(0u, 0u, 0u, 0u);
                vv[u][1] = pj[u] < n ? __ldcg(vp + 1) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        uint32_t bh0 = 0u, bh1 = 0u, bl0 = 0u, bl1 = 0u;
        if (g < nh) {
            bh0 = *reinterpret_cast<const uint32_t*>(&s_ph[g][pb + 2 * t]); bh1 = *reinterpret_cast<const uint32_t*>(&s_ph[g][pb + 2 * t + 8]);
            bl0 = *reinterpret_cast<const uint32_t*>(&s_pl[g][pb + 2 * t]); bl1 = *reinterpret_cast<const uint32_t*>(&s_pl[g][pb + 2 * t + 8]);
        }
        const uint32_t wA[8] = {vv[0][0].x, vv[0][0].y, vv[0][0].z, vv[0][0].w, vv[0][1].x, vv[0][1].y, vv[0][1].z, vv[0][1].w};
        const uint32_t wB[8] = {vv[1][0].x, vv[1][0].y, vv[1][0].z, vv[1][0].w, vv[1][1].x, vv[1][1].y, vv[1][1].z, vv[1][1].w};
        const uint32_t wC[8] = {vv[2][0].x, vv[2][0].y, vv[2][0].z, vv[2][0].w, vv[2][1].x, vv[2][1].y, vv[2][1].z, vv[2][1].w};
        const uint32_t wD[8] = {vv[3][0].x, vv[3][0].y, vv[3][0].z, vv[3][0].w, vv[3][1].x, vv[3][1].y, vv[3][1].z, vv[3][1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // fragment rows g and g + 8 = dims 16 g + 2 i and + 1: the low and the high half of word i; the two
            // positions of a pair come from two rows of the cache
            const uint32_t a0 = __byte_perm(wA[i], wB[i], 0x5410), a1 = __byte_perm(wA[i], wB[i], 0x7632);
            const uint32_t a2 = __byte_perm(wC[i], wD[i], 0x5410), a3 = __byte_perm(wC[i], wD[i], 0x7632);
            mma16816(o[i], a0, a1, a2, a3, bh0, bh1);
            mma16816(o[i], a0, a1, a2, a3, bl0, bl1);
        }
    }
    if (t < 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = 16 * g + 2 * i;
            *reinterpret_cast<float2*>(&s_acc[warp][2 * t][d]) = make_float2(o[i][0], o[i][2]);
            *reinterpret_cast<float2*>(&s_acc[warp][2 * t + 1][d]) = make_float2(o[i][1], o[i][3]);
        }
    }
    __syncthreads();
    for (int hh = 0; hh < nh; ++hh) {
        float* rec = part + ((static_cast<size_t>(b) * H + h0 + hh) * nsplit + split) * (ATT_HD + 2);
        if (threadIdx.x < ATT_HD) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) sum += s_acc[w][hh][threadIdx.x];
            rec[2 + threadIdx.x] = sum;
        }
        if (threadIdx.x == 0) { rec[0] = n > 0 ? s_m[hh] : -INFINITY; rec[1] = n > 0 ? s_l[hh] : 0.f; }
    }
    if (!early) pdl_launch_dependents();
}

template <typename T>
__global__ void __launch_bounds__(ATT_HD) attn_merge_kernel(const float* part, T* out, int nsplit, int early) {
    if (early) pdl_launch_dependents();
    pdl_wait();
    const float* rec = part + static_cast<size_t>(blockIdx.x) * nsplit * (ATT_HD + 2);     // blockIdx.x = b * H + h
    __shared__ float s_w[128];                          // weight of each chunk (nsplit <= 128)
    __shared__ float s_norm;
    // the chunks' maxima and sums, one per thread, then the weights exp2(m_s - m) and the normaliser
    float ms = -INFINITY, ls = 0.f;
    if (static_cast<int>(threadIdx.x) < nsplit) { ms = rec[threadIdx.x * (ATT_HD + 2)]; ls = rec[threadIdx.x * (ATT_HD + 2) + 1]; }
    constexpr int MERGE_PRE = 16;
    const float* col = rec + 2 + threadIdx.x;
    float pre[MERGE_PRE];
#pragma unroll
    for (int u = 0; u < MERGE_PRE; ++u) pre[u] = u < nsplit ? col[static_cast<size_t>(u) * (ATT_HD + 2)] : 0.f;
    float m = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float s_red[4];
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    const float w = ms == -INFINITY ? 0.f : exp2f(ms - m);
    s_w[threadIdx.x] = w;
    float l = w * ls;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = l;
    __syncthreads();
    if (threadIdx.x == 0) s_norm = 1.f / (s_red[0] + s_red[1] + s_red[2] + s_red[3]);
    __syncthreads();
    // thread d: weighted sum of the chunks' dim d. The first 16 chunks were requested before the
    // reductions above (they do not depend on the weights); the rest comes eight at a time, the
    // last batch predicated -- never one dependent load after another.
    float a = 0.f;
#pragma unroll
    for (int u = 0; u < MERGE_PRE; ++u) a = fmaf(u < nsplit ? s_w[u] : 0.f, pre[u], a);
    for (int s = MERGE_PRE; s < nsplit; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = s + u < nsplit ? col[static_cast<size_t>(s + u) * (ATT_HD + 2)] : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u) a = fmaf(s + u < nsplit ? s_w[s + u] : 0.f, v[u], a);
    }
    store_as(out + static_cast<size_t>(blockIdx.x) * ATT_HD + threadIdx.x, a * s_norm);
    if (!early) pdl_launch_dependents();
}

// Launch with programmatic stream serialization (the kernel may start while its predecessor is
// finishing and waits for it itself); TFP8B_NO_PDL=1 in the environment makes it a plain launch.
template <typename... KArgs, typename... Args>
static int launch_pdl(const char* what, void (*kernel)(KArgs...), int grid, int block, cudaStream_t st, Args... args) {
    static const int no_pdl = [] { const char* v = getenv("TFP8B_NO_PDL"); return v && v[0] == '1'; }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(block));
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = no_pdl ? 0 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return cuda_fail(e, what);
    return TFP8B_OK;
}

int glue_status(unsigned int* out, cudaStream_t st) {
    unsigned int* word = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&word), g_status);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(glue status)");
    return read_and_clear_status(word, out, st);
}

// Wait limit of the fused all-reduce, in SM clock cycles. The default, about 17 seconds, is far
// beyond any skew between healthy ranks (a rank's first call can be seconds late: lazy module
// loading, graph instantiation, a garbage-collection pause on its host thread) and still ends the
// kernel if a peer is gone.
static long long g_ar_wait_cycles = 1ll << 35;

// SM count of the current device, asked once per device (148 if the query fails).
static int current_device_sms() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    return sms;
}

// The attention kernels release their dependents when their results are stored, not at once like
// the other helpers: what follows them is the output projection's GEMV, whose weight prefetch
// then competes with the KV cache for HBM -- measured inside a batch-1 decode step of 8 blocks,
// releasing at once costs 13 % of the step (0.94 ms against 0.82). TFP8B_ATT_EARLY=1 restores it.
static int att_early() {
    static const int v = [] { const char* e = getenv("TFP8B_ATT_EARLY"); return (e && e[0] == '1') ? 1 : 0; }();
    return v;
}

static int grid_of(long long work) {
    long long blocks = (work + 255) / 256;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace tfp8b

using namespace tfp8b;

extern "C" int tfp8b_rope_kv_store(const void* qkv, int dtype, const long long* pos, const float* cosv, const float* sinv,
                                   void* q_out, void* k_cache, void* v_cache, int B, int T, int H, int KV, int hd,
                                   int max_seq, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_rope_kv_store: f16 / bf16 only");
    TFP8B_REQUIRE(B >= 0 && T >= 0 && H > 0 && KV > 0 && hd > 0 && hd % 4 == 0 && max_seq > 0, TFP8B_ERR_INVALID,
                  "tfp8b_rope_kv_store: bad shape");
    if (B == 0 || T == 0) return TFP8B_OK;
    TFP8B_REQUIRE(qkv && pos && cosv && sinv && q_out && k_cache && v_cache, TFP8B_ERR_INVALID, "tfp8b_rope_kv_store: null pointer");
    const long long work = static_cast<long long>(B) * T * (H + 2 * KV) * (hd / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TFP8B_F16)
        return launch_pdl("tfp8b_rope_kv_store", rope_kv_kernel<__half>, grid_of(work), 256, st, static_cast<const __half*>(qkv), pos, cosv,
                          sinv, static_cast<__half*>(q_out), static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), B, T, H, KV,
                          hd, max_seq);
    return launch_pdl("tfp8b_rope_kv_store", rope_kv_kernel<__nv_bfloat16>, grid_of(work), 256, st, static_cast<const __nv_bfloat16*>(qkv),
                      pos, cosv, sinv, static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                      static_cast<__nv_bfloat16*>(v_cache), B, T, H, KV, hd, max_seq);
}

template <typename T>
static int rope_kv_fp8_launch(int fmt, int grid, cudaStream_t st, const void* qkv, const long long* pos, const float* cosv,
                              const float* sinv, void* q_out, uint8_t* k_codes, float* k_scale, uint8_t* v_codes, float* v_scale,
                              int B, int Tn, int H, int KV, int max_seq) {
    if (fmt == TFP8B_E4M3FN)
        return launch_pdl("tfp8b_rope_kv_store_fp8", rope_kv_fp8_kernel<T, TFP8B_E4M3FN>, grid, 256, st, static_cast<const T*>(qkv), pos,
                          cosv, sinv, static_cast<T*>(q_out), k_codes, k_scale, v_codes, v_scale, B, Tn, H, KV, max_seq);
    return launch_pdl("tfp8b_rope_kv_store_fp8", rope_kv_fp8_kernel<T, TFP8B_E5M2>, grid, 256, st, static_cast<const T*>(qkv), pos, cosv,
                      sinv, static_cast<T*>(q_out), k_codes, k_scale, v_codes, v_scale, B, Tn, H, KV, max_seq);
}

extern "C" int tfp8b_rope_kv_store_fp8(const void* qkv, int dtype, const long long* pos, const float* cosv, const float* sinv,
                                       void* q_out, uint8_t* k_codes, float* k_scale, uint8_t* v_codes, float* v_scale, int B, int T,
                                       int H, int KV, int hd, int max_seq, int fmt, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_rope_kv_store_fp8: f16 / bf16 only");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_rope_kv_store_fp8: bad fmt %d", fmt);
    TFP8B_REQUIRE(hd == 128, TFP8B_ERR_UNSUPPORTED, "tfp8b_rope_kv_store_fp8: head_dim %d (only 128 is built)", hd);
    TFP8B_REQUIRE(B >= 0 && T >= 0 && H > 0 && KV > 0 && max_seq > 0, TFP8B_ERR_INVALID, "tfp8b_rope_kv_store_fp8: bad shape");
    if (B == 0 || T == 0) return TFP8B_OK;
    TFP8B_REQUIRE(qkv && pos && cosv && sinv && q_out && k_codes && k_scale && v_codes && v_scale, TFP8B_ERR_INVALID,
                  "tfp8b_rope_kv_store_fp8: null pointer");
    const long long work = static_cast<long long>(B) * T * (H + 2 * KV) * 32;      // one warp per head
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TFP8B_F16)
        return rope_kv_fp8_launch<__half>(fmt, grid_of(work), st, qkv, pos, cosv, sinv, q_out, k_codes, k_scale, v_codes, v_scale, B, T,
                                          H, KV, max_seq);
    return rope_kv_fp8_launch<__nv_bfloat16>(fmt, grid_of(work), st, qkv, pos, cosv, sinv, q_out, k_codes, k_scale, v_codes, v_scale, B,
                                             T, H, KV, max_seq);
}

extern "C" int tfp8b_silu_mul(const void* gate_up, void* out, int dtype, long long rows, int F, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_silu_mul: f16 / bf16 only");
    TFP8B_REQUIRE(rows >= 0 && F > 0 && F % 8 == 0, TFP8B_ERR_INVALID, "tfp8b_silu_mul: need F %% 8 == 0");
    if (rows == 0) return TFP8B_OK;
    TFP8B_REQUIRE(gate_up && out, TFP8B_ERR_INVALID, "tfp8b_silu_mul: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long work = rows * (F / 8);
    if (dtype == TFP8B_F16)
        return launch_pdl("tfp8b_silu_mul", silu_mul_kernel<__half>, grid_of(work), 256, st, static_cast<const __half*>(gate_up),
                          static_cast<__half*>(out), rows, F);
    return launch_pdl("tfp8b_silu_mul", silu_mul_kernel<__nv_bfloat16>, grid_of(work), 256, st, static_cast<const __nv_bfloat16*>(gate_up),
                      static_cast<__nv_bfloat16*>(out), rows, F);
}

extern "C" int tfp8b_add_rmsnorm(void* x, const void* delta, const void* weight, void* out, int dtype, long long rows, int dim,
                                 float eps, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_add_rmsnorm: f16 / bf16 only");
    TFP8B_REQUIRE(rows >= 0 && rows <= 0x7fffffffll && dim > 0 && dim % 8 == 0, TFP8B_ERR_INVALID,
                  "tfp8b_add_rmsnorm: need dim %% 8 == 0 and rows < 2^31");
    if (rows == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x && weight && out, TFP8B_ERR_INVALID, "tfp8b_add_rmsnorm: null pointer");
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
                    reinterpret_cast<uintptr_t>(out)) & 15u) == 0, TFP8B_ERR_INVALID, "tfp8b_add_rmsnorm: buffers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TFP8B_F16)
        return launch_pdl("tfp8b_add_rmsnorm", add_rmsnorm_kernel<__half>, static_cast<int>(rows), ADD_NORM_THREADS, st,
                          static_cast<__half*>(x), static_cast<const __half*>(delta), static_cast<const __half*>(weight),
                          static_cast<__half*>(out), dim, eps);
    return launch_pdl("tfp8b_add_rmsnorm", add_rmsnorm_kernel<__nv_bfloat16>, static_cast<int>(rows), ADD_NORM_THREADS, st,
                      static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
                      static_cast<__nv_bfloat16*>(out), dim, eps);
}

extern "C" int tfp8b_attn_decode(const void* q, const void* k_cache, const void* v_cache, const long long* pos, void* out,
                                 float* scratch, long long scratch_floats, int dtype, int B, int H, int KV, int hd, int max_seq,
                                 tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode: f16 / bf16 only");
    TFP8B_REQUIRE(hd == ATT_HD, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode: head_dim %d (only %d is built)", hd, ATT_HD);
    TFP8B_REQUIRE(B >= 0 && H > 0 && KV > 0 && H % KV == 0 && max_seq > 0, TFP8B_ERR_INVALID,
                  "tfp8b_attn_decode: bad shape (H=%d KV=%d)", H, KV);
    if (B == 0) return TFP8B_OK;
    TFP8B_REQUIRE(q && k_cache && v_cache && pos && out && scratch, TFP8B_ERR_INVALID, "tfp8b_attn_decode: null pointer");
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache)) & 15u) == 0, TFP8B_ERR_INVALID,
                  "tfp8b_attn_decode: q and k_cache must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // fp16: both products on the tensor cores, 128 or 256 positions per CTA (TFP8B_ATT16_TC=0: the scalar kernel)
    static const int use_tc = [] { const char* v = getenv("TFP8B_ATT16_TC"); return !(v && v[0] == '0'); }();
    if (use_tc && dtype == TFP8B_F16 && (reinterpret_cast<uintptr_t>(v_cache) & 15u) == 0) {
        const int ngrp_tc = (H / KV + ATT_G - 1) / ATT_G;
        const int sms = current_device_sms();
        const int nw = static_cast<long long>(B) * KV * ngrp_tc * ((max_seq + 127) / 128) >= 2ll * sms ? 8 : 4;
        const int chunk = ATT8_PW * nw, ns = (max_seq + chunk - 1) / chunk;
        TFP8B_REQUIRE(ns <= 128, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode: max_seq %d (at most %d is built)", max_seq, 128 * chunk);
        TFP8B_REQUIRE(scratch_floats >= static_cast<long long>(B) * H * ns * (ATT_HD + 2), TFP8B_ERR_INVALID,
                      "tfp8b_attn_decode: scratch of %lld floats, %lld needed", scratch_floats, static_cast<long long>(B) * H * ns * (ATT_HD + 2));
        const float sl2e = 1.4426950408889634f / sqrtf(static_cast<float>(hd));
        const int grid = B * KV * ngrp_tc * ns;
        const int rc = nw == 8 ? launch_pdl("tfp8b_attn_decode", attn_partial_f16tc_kernel<8>, grid, 256, st, static_cast<const __half*>(q),
                                            static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), pos, scratch, H, KV,
                                            max_seq, ns, sl2e, att_early())
                                : launch_pdl("tfp8b_attn_decode", attn_partial_f16tc_kernel<4>, grid, 128, st, static_cast<const __half*>(q),
                                            static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), pos, scratch, H, KV,
                                            max_seq, ns, sl2e, att_early());
        if (rc != TFP8B_OK) return rc;
        return launch_pdl("tfp8b_attn_decode", attn_merge_kernel<__half>, B * H, ATT_HD, st, static_cast<const float*>(scratch),
                          static_cast<__half*>(out), ns, att_early());
    }
    // chunks of at most ATT_CHUNK positions cover the whole cache
    const int nsplit = (max_seq + ATT_CHUNK - 1) / ATT_CHUNK;
    TFP8B_REQUIRE(nsplit <= 128, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode: max_seq %d (at most %d is built)", max_seq, 128 * ATT_CHUNK);
    const int ngrp = (H / KV + ATT_G - 1) / ATT_G;
    const long long need = static_cast<long long>(B) * H * nsplit * (ATT_HD + 2);
    TFP8B_REQUIRE(scratch_floats >= need, TFP8B_ERR_INVALID, "tfp8b_attn_decode: scratch of %lld floats, %lld needed", scratch_floats, need);
    const float scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(hd));
    int rc;
    if (dtype == TFP8B_F16) {
        rc = launch_pdl("tfp8b_attn_decode", attn_partial_kernel<__half>, B * KV * ngrp * nsplit, ATT_THREADS, st, static_cast<const __half*>(q),
                        static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), pos, scratch, H, KV, max_seq, nsplit,
                        scale_log2e, att_early());
        if (rc != TFP8B_OK) return rc;
        return launch_pdl("tfp8b_attn_decode", attn_merge_kernel<__half>, B * H, ATT_HD, st, static_cast<const float*>(scratch),
                          static_cast<__half*>(out), nsplit, att_early());
    }
    rc = launch_pdl("tfp8b_attn_decode", attn_partial_kernel<__nv_bfloat16>, B * KV * ngrp * nsplit, ATT_THREADS, st,
                    static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
                    static_cast<const __nv_bfloat16*>(v_cache), pos, scratch, H, KV, max_seq, nsplit, scale_log2e, att_early());
    if (rc != TFP8B_OK) return rc;
    return launch_pdl("tfp8b_attn_decode", attn_merge_kernel<__nv_bfloat16>, B * H, ATT_HD, st, static_cast<const float*>(scratch),
                      static_cast<__nv_bfloat16*>(out), nsplit, att_early());
}

template <typename T, int FMT, int NW>
static int attn_fp8_launch_as(int grid, cudaStream_t st, const void* q, const uint8_t* k_codes, const float* k_scale,
                              const uint8_t* v_codes, const float* v_scale, const long long* pos, float* scratch, void* out, int B,
                              int H, int KV, int max_seq, int nsplit, float scale_log2e) {
    const int rc = launch_pdl("tfp8b_attn_decode_fp8", attn_partial_fp8_kernel<T, FMT, NW>, grid, 32 * NW, st, static_cast<const T*>(q),
                              k_codes, k_scale, v_codes, v_scale, pos, scratch, H, KV, max_seq, nsplit, scale_log2e, att_early());
    if (rc != TFP8B_OK) return rc;
    return launch_pdl("tfp8b_attn_decode_fp8", attn_merge_kernel<T>, B * H, ATT_HD, st, static_cast<const float*>(scratch),
                      static_cast<T*>(out), nsplit, att_early());
}

template <typename T>
static int attn_fp8_launch(int fmt, int nw, int grid, cudaStream_t st, const void* q, const uint8_t* k_codes, const float* k_scale,
                           const uint8_t* v_codes, const float* v_scale, const long long* pos, float* scratch, void* out, int B, int H,
                           int KV, int max_seq, int nsplit, float scale_log2e) {
#define ATT8_CASE(F, W) if (fmt == F && nw == W) return attn_fp8_launch_as<T, F, W>(grid, st, q, k_codes, k_scale, v_codes, v_scale, pos, \
                                                                                    scratch, out, B, H, KV, max_seq, nsplit, scale_log2e)
    ATT8_CASE(TFP8B_E4M3FN, 4); ATT8_CASE(TFP8B_E4M3FN, 8); ATT8_CASE(TFP8B_E5M2, 4); ATT8_CASE(TFP8B_E5M2, 8);
#undef ATT8_CASE
    return TFP8B_ERR_INVALID;
}

extern "C" int tfp8b_attn_decode_fp8(const void* q, const uint8_t* k_codes, const float* k_scale, const uint8_t* v_codes,
                                     const float* v_scale, const long long* pos, void* out, float* scratch, long long scratch_floats,
                                     int dtype, int B, int H, int KV, int hd, int max_seq, int fmt, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode_fp8: f16 / bf16 only");
    TFP8B_REQUIRE(fmt == TFP8B_E4M3FN || fmt == TFP8B_E5M2, TFP8B_ERR_INVALID, "tfp8b_attn_decode_fp8: bad fmt %d", fmt);
    TFP8B_REQUIRE(hd == ATT_HD, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode_fp8: head_dim %d (only %d is built)", hd, ATT_HD);
    TFP8B_REQUIRE(B >= 0 && H > 0 && KV > 0 && H % KV == 0 && max_seq > 0, TFP8B_ERR_INVALID,
                  "tfp8b_attn_decode_fp8: bad shape (H=%d KV=%d)", H, KV);
    if (B == 0) return TFP8B_OK;
    TFP8B_REQUIRE(q && k_codes && k_scale && v_codes && v_scale && pos && out && scratch, TFP8B_ERR_INVALID,
                  "tfp8b_attn_decode_fp8: null pointer");
    TFP8B_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_codes)) & 15u) == 0 &&
                  (reinterpret_cast<uintptr_t>(v_codes) & 15u) == 0, TFP8B_ERR_INVALID,
                  "tfp8b_attn_decode_fp8: q, k_codes and v_codes must be 16-byte aligned");
    const int ngrp = (H / KV + ATT_G - 1) / ATT_G;
    // 128 positions per CTA (four warps) while that leaves the machine short of CTAs, 256 (eight warps)
    // beyond: half the partial records and half the merge work (prompt 2100: 10.0 -> 9.5 us per call
    // at batch 4, 17.2 -> 16.4 at batch 8). TFP8B_ATT8_WARPS=4|8 forces one.
    static const int nw_env = [] { const char* v = getenv("TFP8B_ATT8_WARPS"); return v ? atoi(v) : 0; }();
    const int sms = current_device_sms();
    const long long ctas128 = static_cast<long long>(B) * KV * ngrp * ((max_seq + 127) / 128);
    const int nw = (nw_env == 4 || nw_env == 8) ? nw_env : (ctas128 >= 2ll * sms ? 8 : 4);
    const int chunk = ATT8_PW * nw;
    const int nsplit = (max_seq + chunk - 1) / chunk;
    TFP8B_REQUIRE(nsplit <= 128, TFP8B_ERR_UNSUPPORTED, "tfp8b_attn_decode_fp8: max_seq %d (at most %d is built)", max_seq, 128 * chunk);
    const long long need = static_cast<long long>(B) * H * nsplit * (ATT_HD + 2);
    TFP8B_REQUIRE(scratch_floats >= need, TFP8B_ERR_INVALID, "tfp8b_attn_decode_fp8: scratch of %lld floats, %lld needed", scratch_floats, need);
    const float scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(hd));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = B * KV * ngrp * nsplit;
    if (dtype == TFP8B_F16)
        return attn_fp8_launch<__half>(fmt, nw, grid, st, q, k_codes, k_scale, v_codes, v_scale, pos, scratch, out, B, H, KV, max_seq, nsplit,
                                       scale_log2e);
    return attn_fp8_launch<__nv_bfloat16>(fmt, nw, grid, st, q, k_codes, k_scale, v_codes, v_scale, pos, scratch, out, B, H, KV, max_seq,
                                          nsplit, scale_log2e);
}

extern "C" int tfp8b_allreduce_add_rmsnorm(void* x, const float* partial, const void* weight, void* out, int dtype, int rows,
                                           int dim, float eps, float* const* recv, unsigned int* const* flags,
                                           unsigned int* state, int rank, int world, int max_rows, tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_allreduce_add_rmsnorm: f16 / bf16 only");
    TFP8B_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, TFP8B_ERR_INVALID,
                  "tfp8b_allreduce_add_rmsnorm: rank %d of %d (1..8 ranks)", rank, world);
    TFP8B_REQUIRE(rows >= 0 && rows <= max_rows && dim > 0 && dim % 4 == 0 && dim <= 4 * AR_THREADS * 4, TFP8B_ERR_INVALID,
                  "tfp8b_allreduce_add_rmsnorm: rows=%d (receive area holds %d), dim=%d (a multiple of 4, at most %d)", rows,
                  max_rows, dim, 4 * AR_THREADS * 4);
    if (rows == 0) return TFP8B_OK;
    TFP8B_REQUIRE(x && partial && weight && out && recv && flags && state, TFP8B_ERR_INVALID, "tfp8b_allreduce_add_rmsnorm: null pointer");
    ArParams ar;
    for (int r = 0; r < 8; ++r) {
        ar.recv[r] = r < world ? recv[r] : nullptr;
        ar.flag[r] = r < world ? flags[r] : nullptr;
        if (r < world) TFP8B_REQUIRE(ar.recv[r] && ar.flag[r], TFP8B_ERR_INVALID, "tfp8b_allreduce_add_rmsnorm: null peer pointer %d", r);
    }
    ar.state = state; ar.rank = rank; ar.world = world; ar.max_rows = max_rows;
    ar.wait_cycles = __atomic_load_n(&g_ar_wait_cycles, __ATOMIC_RELAXED);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TFP8B_F16)
        return launch_pdl("tfp8b_allreduce_add_rmsnorm", allreduce_add_rmsnorm_kernel<__half>, rows, AR_THREADS, st,
                          static_cast<__half*>(x), partial, static_cast<const __half*>(weight), static_cast<__half*>(out), dim, eps, ar);
    return launch_pdl("tfp8b_allreduce_add_rmsnorm", allreduce_add_rmsnorm_kernel<__nv_bfloat16>, rows, AR_THREADS, st,
                      static_cast<__nv_bfloat16*>(x), partial, static_cast<const __nv_bfloat16*>(weight),
                      static_cast<__nv_bfloat16*>(out), dim, eps, ar);
}

extern "C" long long tfp8b_allreduce_wait_limit(long long cycles) {
    const long long old = __atomic_load_n(&g_ar_wait_cycles, __ATOMIC_RELAXED);
    if (cycles > 0) __atomic_store_n(&g_ar_wait_cycles, cycles, __ATOMIC_RELAXED);
    return old;
}

extern "C" int tfp8b_argmax(const void* logits, int dtype, long long* out, long long rows, long long n, long long row_pitch,
                            tfp8b_stream_t stream) {
    TFP8B_REQUIRE(dtype == TFP8B_F16 || dtype == TFP8B_BF16, TFP8B_ERR_UNSUPPORTED, "tfp8b_argmax: f16 / bf16 only");
    TFP8B_REQUIRE(rows >= 0 && rows <= 0x7fffffffll && n > 0 && row_pitch >= n, TFP8B_ERR_INVALID, "tfp8b_argmax: bad shape");
    if (rows == 0) return TFP8B_OK;
    TFP8B_REQUIRE(logits && out, TFP8B_ERR_INVALID, "tfp8b_argmax: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == TFP8B_F16)
        return launch_pdl("tfp8b_argmax", argmax_kernel<__half>, static_cast<int>(rows), ARGMAX_THREADS, st,
                          static_cast<const __half*>(logits), out, n, row_pitch);
    return launch_pdl("tfp8b_argmax", argmax_kernel<__nv_bfloat16>, static_cast<int>(rows), ARGMAX_THREADS, st,
                      static_cast<const __nv_bfloat16*>(logits), out, n, row_pitch);
}
