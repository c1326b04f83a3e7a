// Memory-bound glue of the transformer layers: RMSNorm (zero-centred gain), the sandwich-norm
// residual update, QK-norm + rotary embedding, the scaled token embedding, the judgment
// head and the per-question candidate softmax.  All kernels move 16 bytes per thread per
// access, keep a row in registers between the reduction and the write, and reduce with
// warp shuffles; the roofline that bounds them is HBM bandwidth.
#include "common.cuh"

namespace {

using namespace bg;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 v;
    v.x = pack_bf16(f[0], f[1]);
    v.y = pack_bf16(f[2], f[3]);
    v.z = pack_bf16(f[4], f[5]);
    v.w = pack_bf16(f[6], f[7]);
    return v;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Block-wide sum; every thread receives the total.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();   // scratch may still be read from a previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < warps ? scratch[lane] : 0.f;
    return warp_sum(t);
}

// Store 8 consecutive values of a row (columns c..c+7, already rounded to bf16) as MXFP8: the four threads
// that share a 32-element block agree on its power-of-two scale through two shuffles.  Every thread of the
// warp must call this (inactive ones with zeros).
__device__ __forceinline__ void store_mxfp8(const float* f, bool active, uint8_t* q, uint8_t* sf, int64_t row, int c,
                                            int h) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!active) return;
    const int e = mx_exponent(amax);
    const float inv = exp2f(float(-e));
    uint2 o;
    o.x = e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
    o.y = e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
    *reinterpret_cast<uint2*>(q + row * h + c) = o;
    if ((c & 31) == 0) sf[mx_scale_offset(row, c >> 5, h >> 7)] = uint8_t(e + 127);
}

// out = rmsnorm(x) * (1 + w).  One block per row, one 16-byte chunk per thread.
// Restates transformers T5Gemma2RMSNorm (modeling_t5gemma2.py:61-69): fp32 math, the gain is
// applied before the result is rounded to bf16.
// With out_q / out_sf the result is written as MXFP8 (contiguous [rows, h] values + scale atoms) instead of bf16.
__global__ void rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w,
                               __nv_bfloat16* __restrict__ out, int64_t ldo, int h, float eps,
                               uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int64_t row = blockIdx.x;
    const int c = threadIdx.x * 8;
    float f[8];
    const bool active = c < h;
    float ss = 0.f;
    if (active) {
        unpack8(*reinterpret_cast<const uint4*>(x + row * ldx + c), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    const float r = rsqrtf(block_sum(ss, scratch) / float(h) + eps);
    if (active) {
        float g[8];
        unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * r * (1.f + g[i]);
        if (out_q == nullptr) *reinterpret_cast<uint4*>(out + row * ldo + c) = pack8(f);
    }
    if (out_q != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = active ? round_bf16(f[i]) : 0.f;
        store_mxfp8(f, active, out_q, out_sf, row, c, h);
    }
}

// Sandwich-norm residual update fused with the next pre-norm:
//   resid <- resid + bf16(rmsnorm(y) * (1 + w_post));   normed <- rmsnorm(resid) * (1 + w_next)
// (transformers modeling_t5gemma2.py:496-502: post-norm, residual add, then the next block's
// pre-norm).  The rounding points of the bf16 module chain are kept: the post-norm output
// and the updated residual are each rounded to bf16 before they are used again.
// w_next == nullptr skips the second norm.
__global__ void add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ w_post,
                                   __nv_bfloat16* __restrict__ resid, const __nv_bfloat16* __restrict__ w_next,
                                   __nv_bfloat16* __restrict__ normed, int h, float eps,
                                   uint8_t* __restrict__ normed_q, uint8_t* __restrict__ normed_sf) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int64_t row = blockIdx.x;
    const int c = threadIdx.x * 8;
    const bool active = c < h;
    float f[8], x[8];
    float ss = 0.f;
    // both row loads are issued before the first reduction so that two 16-byte requests per
    // thread are in flight; y is read exactly once (streaming load)
    uint4 raw_y = make_uint4(0, 0, 0, 0), raw_x = make_uint4(0, 0, 0, 0), raw_g = make_uint4(0, 0, 0, 0);
    if (active) {
        raw_y = __ldcs(reinterpret_cast<const uint4*>(y + row * h + c));
        raw_x = *reinterpret_cast<const uint4*>(resid + row * h + c);
        raw_g = __ldg(reinterpret_cast<const uint4*>(w_post + c));
        unpack8(raw_y, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    float r = rsqrtf(block_sum(ss, scratch) / float(h) + eps);
    ss = 0.f;
    if (active) {
        float g[8];
        unpack8(raw_g, g);
        unpack8(raw_x, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            x[i] = round_bf16(x[i] + round_bf16(f[i] * r * (1.f + g[i])));
            ss += x[i] * x[i];
        }
        *reinterpret_cast<uint4*>(resid + row * h + c) = pack8(x);
    }
    if (w_next == nullptr) return;
    r = rsqrtf(block_sum(ss, scratch) / float(h) + eps);
    if (active) {
        float g[8];
        unpack8(*reinterpret_cast<const uint4*>(w_next + c), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = x[i] * r * (1.f + g[i]);
        if (normed_q == nullptr) *reinterpret_cast<uint4*>(normed + row * h + c) = pack8(x);
    }
    if (normed_q != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = active ? round_bf16(x[i]) : 0.f;
        store_mxfp8(x, active, normed_q, normed_sf, row, c, h);
    }
}


// ---------------------------------------------------------------- row-per-warp norm kernels
// For hidden sizes that are a multiple of 256 (CH chunks of 32 lanes x 8 elements) one WARP owns a
// row: it issues every 16-byte load of the row (and of the residual row) before the first use, so
// a lane keeps CH (2 CH, 3 CH) independent requests in flight, reduces with shuffles only - no
// shared memory, no block barrier - and walks on to row + (warps in the grid).  The residual stream
// may be bf16 (the module chain's own rounding points are kept) or fp32 (no rounding between layers).
template <typename T>
struct Chunk8;
template <>
struct Chunk8<__nv_bfloat16> {
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void load_streaming(const __nv_bfloat16* p) { v = __ldcs(reinterpret_cast<const uint4*>(p)); }
    __device__ __forceinline__ void get(float* f) const { unpack8(v, f); }
    __device__ __forceinline__ void set(const float* f) { v = pack8(f); }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = v; }
};
template <>
struct Chunk8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = reinterpret_cast<const float4*>(p)[0];
        b = reinterpret_cast<const float4*>(p)[1];
    }
    __device__ __forceinline__ void load_streaming(const float* p) { load(p); }
    __device__ __forceinline__ void get(float* f) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    __device__ __forceinline__ void set(const float* f) {
        a = make_float4(f[0], f[1], f[2], f[3]);
        b = make_float4(f[4], f[5], f[6], f[7]);
    }
    __device__ __forceinline__ void store(float* p) const {
        reinterpret_cast<float4*>(p)[0] = a;
        reinterpret_cast<float4*>(p)[1] = b;
    }
};
template <typename T> __device__ __forceinline__ float round_as(float x);
template <> __device__ __forceinline__ float round_as<__nv_bfloat16>(float x) { return round_bf16(x); }
template <> __device__ __forceinline__ float round_as<float>(float x) { return x; }

constexpr int ROW_WARPS = 4;    // warps per block of the row-per-warp kernels

template <int CH, typename XT>
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_rows_kernel(const XT* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w,
                    __nv_bfloat16* __restrict__ out, int64_t ldo, int64_t rows, float eps,
                    uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t stride = int64_t(gridDim.x) * ROW_WARPS;
    constexpr float inv_h = 1.f / float(CH * 256);
    for (int64_t row = int64_t(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5); row < rows; row += stride) {
        Chunk8<XT> xv[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) xv[c].load_streaming(x + row * ldx + c * 256 + lane * 8);
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float f[8];
            xv[c].get(f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
        }
        const float r = rsqrtf(warp_sum(ss) * inv_h + eps);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float f[8], g[8];
            xv[c].get(f);
            unpack8(__ldg(reinterpret_cast<const uint4*>(w + c * 256 + lane * 8)), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = f[i] * r * (1.f + g[i]);
            if (out_q == nullptr) {
                *reinterpret_cast<uint4*>(out + row * ldo + c * 256 + lane * 8) = pack8(f);
            } else {        // MXFP8 of the bf16-rounded row: four neighbouring lanes share a 32-element block
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = round_bf16(f[i]);
                store_mxfp8(f, true, out_q, out_sf, row, c * 256 + lane * 8, CH * 256);
            }
        }
    }
}

// resid <- resid + post_norm(y);  normed <- pre_norm(resid)   (see add_rmsnorm_kernel for the contract).
// RT = __nv_bfloat16: post-norm result and updated residual are each rounded to bf16, as the module chain does;
// RT = float: the residual stream stays in fp32 and nothing is rounded on the way into it.
template <int CH, typename RT, typename YT>
__global__ void __launch_bounds__(ROW_WARPS * 32)
add_rmsnorm_rows_kernel(const YT* __restrict__ y, const __nv_bfloat16* __restrict__ w_post,
                        RT* __restrict__ resid, const __nv_bfloat16* __restrict__ w_next,
                        __nv_bfloat16* __restrict__ normed, int64_t rows, float eps,
                        uint8_t* __restrict__ normed_q, uint8_t* __restrict__ normed_sf) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t stride = int64_t(gridDim.x) * ROW_WARPS;
    constexpr int H = CH * 256;
    constexpr float inv_h = 1.f / float(H);
    for (int64_t row = int64_t(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5); row < rows; row += stride) {
        Chunk8<YT> yv[CH];
        Chunk8<RT> xv[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) yv[c].load_streaming(y + row * H + c * 256 + lane * 8);
#pragma unroll
        for (int c = 0; c < CH; ++c) xv[c].load(resid + row * H + c * 256 + lane * 8);
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float f[8];
            yv[c].get(f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
        }
        float r = rsqrtf(warp_sum(ss) * inv_h + eps);
        ss = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float f[8], g[8], x[8];
            yv[c].get(f);
            xv[c].get(x);
            unpack8(__ldg(reinterpret_cast<const uint4*>(w_post + c * 256 + lane * 8)), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x[i] = round_as<RT>(x[i] + round_as<RT>(f[i] * r * (1.f + g[i])));
                ss += x[i] * x[i];
            }
            xv[c].set(x);
            xv[c].store(resid + row * H + c * 256 + lane * 8);
        }
        if (w_next == nullptr) continue;
        r = rsqrtf(warp_sum(ss) * inv_h + eps);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float x[8], g[8];
            xv[c].get(x);
            unpack8(__ldg(reinterpret_cast<const uint4*>(w_next + c * 256 + lane * 8)), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = x[i] * r * (1.f + g[i]);
            if (normed_q == nullptr) {
                *reinterpret_cast<uint4*>(normed + row * H + c * 256 + lane * 8) = pack8(x);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = round_bf16(x[i]);
                store_mxfp8(x, true, normed_q, normed_sf, row, c * 256 + lane * 8, H);
            }
        }
    }
}

// QK-norm + RoPE in place.  One warp per token walks that token's query heads and key heads:
// per head an fp32 RMSNorm over head_dim with (1 + w) gain, then rotate-half RoPE with the
// angle position * inv_freq[i mod D/2] (bongard/attention.py:172-180; the fused form follows
// bongard/qk_norm_rope.metal:4-33: partner j = (i + D/2) mod D, sign - for i < D/2).
// Lane l owns HE = D/64 elements of the FIRST half, [l*HE, (l+1)*HE), and their rotation partners in the
// second half, [D/2 + l*HE, ...): both members of a pair sit in one lane, so the rotation needs no shuffle
// and every angle is computed once (not once per half).  Heads are taken four at a time: the eight loads
// of a batch are issued before the first is used, which is what keeps enough bytes in flight.
// rotate == 0 leaves out the rotation (decoder state keys: bongard/model.py:135-139).
template <int HE>
struct HalfVec;          // HE bf16 values as one load
template <> struct HalfVec<4> { using T = uint2; };
template <> struct HalfVec<2> { using T = uint32_t; };
template <> struct HalfVec<1> { using T = uint16_t; };

template <int HE>
__device__ __forceinline__ void unpack_half(const typename HalfVec<HE>::T& raw, float* f) {
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int e = 0; e < HE; ++e) f[e] = __bfloat162float(h[e]);
}
template <int HE>
__device__ __forceinline__ typename HalfVec<HE>::T pack_half(const float* f) {
    typename HalfVec<HE>::T raw;
    __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
    for (int e = 0; e < HE; ++e) h[e] = __float2bfloat16_rn(f[e]);
    return raw;
}

template <int D>
__global__ void qk_norm_rope_kernel(__nv_bfloat16* __restrict__ q, int64_t ldq, int q_heads,
                                    __nv_bfloat16* __restrict__ k, int64_t ldk, int k_heads,
                                    const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                    const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                    const __nv_bfloat16* __restrict__ cos_table,
                                    const __nv_bfloat16* __restrict__ sin_table,
                                    const float2* __restrict__ angle_table, int angle_rows, int64_t tokens, float eps,
                                    int rotate) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int HE = D / 64;     // elements per lane and half
    constexpr int NB = 4;          // heads per batch
    using Vec = typename HalfVec<HE>::T;
    const int lane = threadIdx.x & 31;
    const int64_t token = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= tokens) return;
    if (k == nullptr) k_heads = 0;
    const int first = lane * HE;           // this lane's columns: [first, first + HE) and D/2 + the same
    float cs[HE], sn[HE], cs2[HE], sn2[HE];     // angles of the first-half columns and of their partners
    if (rotate && cos_table != nullptr) {
        // caller-supplied tables [tokens, D] (the rotary module's cos/sin, cat(freqs, freqs))
#pragma unroll
        for (int e = 0; e < HE; ++e) {
            cs[e] = __bfloat162float(cos_table[token * D + first + e]);
            sn[e] = __bfloat162float(sin_table[token * D + first + e]);
            cs2[e] = __bfloat162float(cos_table[token * D + D / 2 + first + e]);
            sn2[e] = __bfloat162float(sin_table[token * D + D / 2 + first + e]);
        }
    } else if (rotate && angle_table != nullptr) {
        // (cos, sin) of position * inv_freq, computed once per position by rope_table_kernel with the same
        // expression as below: the same bits without 4 sincosf per lane and token
        int pos = positions[token];
        pos = pos < 0 ? 0 : (pos >= angle_rows ? angle_rows - 1 : pos);
        const float2* row = angle_table + int64_t(pos) * (D / 2) + first;
#pragma unroll
        for (int e = 0; e < HE; ++e) {
            const float2 a = __ldg(row + e);
            cs[e] = cs2[e] = a.x;
            sn[e] = sn2[e] = a.y;
        }
    } else if (rotate) {
        const float pos = float(positions[token]);
#pragma unroll
        for (int e = 0; e < HE; ++e) {
            sincosf(pos * inv_freq[first + e], &sn[e], &cs[e]);
            cs2[e] = cs[e];
            sn2[e] = sn[e];
        }
    }
    // gains of this lane's columns (q and k), as 1 + w
    float gq[2][HE], gk[2][HE];
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int e = 0; e < HE; ++e) {
            gq[half][e] = q_heads ? 1.f + __bfloat162float(qw[half * (D / 2) + first + e]) : 1.f;
            gk[half][e] = k_heads ? 1.f + __bfloat162float(kw[half * (D / 2) + first + e]) : 1.f;
        }
    const int heads = q_heads + k_heads;
    for (int base = 0; base < heads; base += NB) {
        Vec raw[NB][2];
        __nv_bfloat16* ptr[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int head = base + b;
            if (head < heads) {
                ptr[b] = (head < q_heads ? q + token * ldq + head * D : k + token * ldk + (head - q_heads) * D) + first;
                raw[b][0] = *reinterpret_cast<const Vec*>(ptr[b]);
                raw[b][1] = *reinterpret_cast<const Vec*>(ptr[b] + D / 2);
            }
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int head = base + b;
            if (head >= heads) break;
            const bool is_q = head < q_heads;
            float x1[HE], x2[HE];
            unpack_half<HE>(raw[b][0], x1);
            unpack_half<HE>(raw[b][1], x2);
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < HE; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
            const float r = rsqrtf(warp_sum(ss) / float(D) + eps);
#pragma unroll
            for (int e = 0; e < HE; ++e) {
                x1[e] = x1[e] * r * (is_q ? gq[0][e] : gk[0][e]);
                x2[e] = x2[e] * r * (is_q ? gq[1][e] : gk[1][e]);
            }
            if (rotate) {
#pragma unroll
                for (int e = 0; e < HE; ++e) {
                    const float a = x1[e], c = x2[e];
                    x1[e] = a * cs[e] - c * sn[e];
                    x2[e] = c * cs2[e] + a * sn2[e];
                }
            }
            *reinterpret_cast<Vec*>(ptr[b]) = pack_half<HE>(x1);
            *reinterpret_cast<Vec*>(ptr[b] + D / 2) = pack_half<HE>(x2);
        }
    }
}

// (cos, sin) of position * inv_freq[i] for every position below `rows`, the angles the QK-norm + RoPE
// kernel computes on the fly; the q|k|v GEMM epilogue reads them from this table instead.
__global__ void rope_table_kernel(float2* __restrict__ table, int64_t rows, int half, const float* __restrict__ inv_freq) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * half) return;
    const float pos = float(i / half);
    float sn, cs;
    sincosf(pos * inv_freq[i % half], &sn, &cs);
    table[i] = make_float2(cs, sn);
}

// Scaled word embedding with the end-of-image override (transformers modeling_t5gemma2.py:644-647).
// OT = float writes the fp32 residual stream: the product table * scale is then not rounded.
template <typename OT>
__global__ void embed_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             const __nv_bfloat16* __restrict__ eoi, OT* __restrict__ out, int h,
                             float scale, int64_t eoi_token, int64_t vocab) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t row = blockIdx.x;
    const int c = threadIdx.x * 8;
    if (c >= h) return;
    int64_t id = ids[row];
    float f[8];
    if (id == eoi_token) {
        unpack8(*reinterpret_cast<const uint4*>(eoi + c), f);
    } else {
        if (id < 0 || id >= vocab) id = 0;
        unpack8(*reinterpret_cast<const uint4*>(table + id * h + c), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= scale;
    }
    Chunk8<OT> v;
    v.set(f);
    v.store(out + row * h + c);
}

// Judgment head (bongard/model.py:92-95): logit = w.h + (C h).(G g) / sqrt(rank).
// A cluster of HEAD_SPLIT CTAs per candidate: CTA r takes rows [r, r+1) * rank/HEAD_SPLIT of C and G,
// one warp per row with the lanes striding along it (coalesced 512-byte reads), and parks its partial
// sum in shared memory; CTA 0 adds the partials in rank order through distributed shared memory, so
// the result does not depend on scheduling.  A single question (2-10 candidates) thereby spreads the
// 2.6 MB of head weights over 16-80 SMs instead of 2-10.  fp32 throughout.
constexpr int HEAD_SPLIT = 8;

__global__ void __cluster_dims__(1, HEAD_SPLIT, 1)
judgment_head_kernel(const __nv_bfloat16* __restrict__ hidden, int64_t ldh,
                     const int32_t* __restrict__ cand_rows, const int32_t* __restrict__ dec_rows,
                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ cmat,
                     const __nv_bfloat16* __restrict__ gmat, float* __restrict__ logits, int h,
                     int rank) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float sh[];      // h floats of the candidate row, h floats of the decision row
    __shared__ float scratch[33];
    __shared__ float warp_acc[8];
    __shared__ float partial;
    float* hc = sh;
    float* hg = sh + h;
    const int cand = blockIdx.x;
    const int chunk = blockIdx.y;      // == rank of this CTA in its cluster
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const __nv_bfloat16* pc = hidden + int64_t(cand_rows[cand]) * ldh;
    const __nv_bfloat16* pg = hidden + int64_t(dec_rows[cand]) * ldh;
    for (int i = threadIdx.x * 8; i < h; i += blockDim.x * 8) {
        unpack8(*reinterpret_cast<const uint4*>(pc + i), hc + i);
        unpack8(*reinterpret_cast<const uint4*>(pg + i), hg + i);
    }
    __syncthreads();
    const int per = (rank + HEAD_SPLIT - 1) / HEAD_SPLIT;
    const int j_hi = min(rank, (chunk + 1) * per);
    float acc = 0.f;
    for (int j = chunk * per + warp; j < j_hi; j += warps) {
        const __nv_bfloat16* cr = cmat + int64_t(j) * h;
        const __nv_bfloat16* gr = gmat + int64_t(j) * h;
        float a = 0.f, b = 0.f;
        for (int i = lane * 8; i < h; i += 256) {
            float fc[8], fg[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(cr + i)), fc);
            unpack8(__ldg(reinterpret_cast<const uint4*>(gr + i)), fg);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a += fc[e] * hc[i + e];
                b += fg[e] * hg[i + e];
            }
        }
        a = warp_sum(a);
        b = warp_sum(b);
        acc += a * b;                  // identical in every lane
    }
    if (lane == 0) warp_acc[warp] = acc;
    float wdot = 0.f;
    if (chunk == 0) {
        float t = 0.f;
        for (int i = threadIdx.x; i < h; i += blockDim.x) t += __bfloat162float(w[i]) * hc[i];
        wdot = block_sum(t, scratch);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int k = 0; k < warps; ++k) t += warp_acc[k];
        partial = t;
    }
    bg::cluster_sync();                // every CTA's partial is written and visible
    if (chunk == 0 && threadIdx.x == 0) {
        float total = 0.f;
        const uint32_t addr = bg::smem_u32(&partial);
        for (int r = 0; r < HEAD_SPLIT; ++r) {
            float v;
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(bg::map_to_cta(addr, (uint32_t)r)));
            total += v;
        }
        logits[cand] = total * rsqrtf(float(rank)) + wdot;
    }
    bg::cluster_sync();                // no CTA leaves while CTA 0 reads its partial
}

// dst[c, r] = src[r, c] for a bf16 matrix, through a padded 64 x 64 shared-memory tile so that both the
// reads and the writes are coalesced.  Feeds the backward of the linears: the tensor-core GEMM takes both
// operands K-contiguous, and dX = dY W / dW = dY^T X contract over the dimension that is NOT contiguous
// in W, dY and X.
__global__ void transpose_kernel(const __nv_bfloat16* __restrict__ src, int64_t lds, __nv_bfloat16* __restrict__ dst,
                                 int64_t ldd, int64_t rows, int64_t cols) {
    __shared__ __nv_bfloat16 tile[64][66];
    const int64_t r0 = int64_t(blockIdx.y) * 64, c0 = int64_t(blockIdx.x) * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;     // 256 threads: 64 columns x 4 rows per pass
    for (int i = ty; i < 64; i += 4) {
        const int64_t r = r0 + i, c = c0 + tx;
        tile[i][tx] = (r < rows && c < cols) ? src[r * lds + c] : __float2bfloat16(0.f);
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 4) {
        const int64_t c = c0 + i, r = r0 + tx;
        if (c < cols && r < rows) dst[c * ldd + r] = tile[tx][i];
    }
}

// Backward of the GeGLU epilogue h = gelu_tanh(g) * u for gu = [g | u] (both [rows, inter], bf16):
// dgu = [dh * u * gelu_tanh'(g) | dh * gelu_tanh(g)].
__global__ void geglu_backward_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                      __nv_bfloat16* __restrict__ dgu, int64_t rows, int64_t inter) {
    const int64_t i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * inter) return;
    const int64_t row = i / inter, col = i % inter;             // inter % 8 == 0: the 8 elements share a row
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + row * 2 * inter + col), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter + col), u);
    unpack8(*reinterpret_cast<const uint4*>(dh + i), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float k0 = 0.7978845608028654f, k1 = 0.044715f;
        const float x = g[e];
        const float t = tanhf(k0 * (x + k1 * x * x * x));
        const float gelu = 0.5f * x * (1.f + t);
        const float dgelu = 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
        dg[e] = d[e] * u[e] * dgelu;
        du[e] = d[e] * gelu;
    }
    *reinterpret_cast<uint4*>(dgu + row * 2 * inter + col) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + row * 2 * inter + inter + col) = pack8(du);
}

// Per-question temperature softmax in float64 (bongard/inference.py:54-73), one thread per question.
__global__ void candidate_softmax_kernel(const float* __restrict__ logits, const int32_t* __restrict__ offsets,
                                         double* __restrict__ probs, int questions, double temperature) {
    pdl_wait();
    pdl_launch_dependents();
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= questions) return;
    const int lo = offsets[q], hi = offsets[q + 1];
    if (hi <= lo) return;
    double zmax = -INFINITY;
    for (int i = lo; i < hi; ++i) {
        double z = double(logits[i]);
        if (temperature >= 1.0) z /= temperature;
        zmax = fmax(zmax, z);
    }
    double sum = 0.0;
    for (int i = lo; i < hi; ++i) {
        double z = double(logits[i]);
        z = temperature >= 1.0 ? z / temperature - zmax : (z - zmax) / temperature;
        const double e = exp(z);
        probs[i] = e;
        sum += e;
    }
    double total = 0.0;
    for (int i = lo; i < hi; ++i) {
        probs[i] /= sum;
        total += probs[i];
    }
    for (int i = lo; i < hi; ++i) probs[i] /= total;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        bg_set_error("%s: launch: %s", what, cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

int row_threads(int64_t h) { return int(((h / 8 + 31) / 32) * 32); }

// Grid of the row-per-warp kernels: enough blocks for every row, at most 16 per SM (rows beyond that are
// reached by the stride loop).
unsigned row_grid(int64_t rows) {
    const int64_t blocks = (rows + ROW_WARPS - 1) / ROW_WARPS;
    const int64_t cap = int64_t(bg_num_sms()) * 16;
    return (unsigned)(blocks < cap ? blocks : cap);
}

// Row-per-warp RMSNorm for hidden sizes 256 * {1..16}; false when the size is not covered.
template <typename XT>
bool launch_rmsnorm_rows(const XT* x, int64_t ldx, const __nv_bfloat16* w, __nv_bfloat16* out, int64_t ldo, int64_t rows,
                         int64_t h, float eps, cudaStream_t s, uint8_t* out_q = nullptr, uint8_t* out_sf = nullptr) {
    if (h % 256 || h > 4096) return false;
    const dim3 grid(row_grid(rows)), block(ROW_WARPS * 32);
#define BG_ROWS_CASE(CH) case CH: launch_kernel(rmsnorm_rows_kernel<CH, XT>, grid, block, 0, s, 0, x, ldx, w, out, ldo, rows, eps, out_q, out_sf); return true;
    switch (int(h / 256)) {
        BG_ROWS_CASE(1) BG_ROWS_CASE(2) BG_ROWS_CASE(3) BG_ROWS_CASE(4) BG_ROWS_CASE(5) BG_ROWS_CASE(6) BG_ROWS_CASE(7) BG_ROWS_CASE(8)
        BG_ROWS_CASE(9) BG_ROWS_CASE(10) BG_ROWS_CASE(11) BG_ROWS_CASE(12) BG_ROWS_CASE(13) BG_ROWS_CASE(14) BG_ROWS_CASE(15) BG_ROWS_CASE(16)
    }
#undef BG_ROWS_CASE
    return false;
}

template <typename RT, typename YT>
bool launch_add_rmsnorm_rows(const YT* y, const __nv_bfloat16* w_post, RT* resid, const __nv_bfloat16* w_next,
                             __nv_bfloat16* normed, int64_t rows, int64_t h, float eps, cudaStream_t s,
                             uint8_t* normed_q = nullptr, uint8_t* normed_sf = nullptr) {
    if (h % 256 || h > 4096 || (sizeof(YT) == 4 && h > 3072)) return false;
    const dim3 grid(row_grid(rows)), block(ROW_WARPS * 32);
#define BG_ROWS_CASE(CH) case CH: launch_kernel(add_rmsnorm_rows_kernel<CH, RT, YT>, grid, block, 0, s, 0, y, w_post, resid, w_next, normed, rows, eps, normed_q, normed_sf); return true;
    switch (int(h / 256)) {
        BG_ROWS_CASE(1) BG_ROWS_CASE(2) BG_ROWS_CASE(3) BG_ROWS_CASE(4) BG_ROWS_CASE(5) BG_ROWS_CASE(6) BG_ROWS_CASE(7) BG_ROWS_CASE(8)
        BG_ROWS_CASE(9) BG_ROWS_CASE(10) BG_ROWS_CASE(11) BG_ROWS_CASE(12) BG_ROWS_CASE(13) BG_ROWS_CASE(14) BG_ROWS_CASE(15) BG_ROWS_CASE(16)
    }
#undef BG_ROWS_CASE
    return false;
}

}  // namespace

extern "C" {

int bg_rmsnorm(const void* x, int64_t ldx, const void* w, void* out, int64_t ldo, int64_t rows, int64_t h,
               float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 8 || h > 8192 || ldx % 8 || ldo % 8) {
        bg_set_error("bg_rmsnorm: hidden size must be a multiple of 8 up to 8192 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    if (launch_rmsnorm_rows(static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w),
                            static_cast<__nv_bfloat16*>(out), ldo, rows, h, eps, static_cast<cudaStream_t>(stream)))
        return check_launch("bg_rmsnorm");
    launch_kernel(rmsnorm_kernel, dim3((unsigned)rows), dim3(row_threads(h)), 0, static_cast<cudaStream_t>(stream), 0,
                  static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w),
                  static_cast<__nv_bfloat16*>(out), ldo, (int)h, eps, (uint8_t*)nullptr, (uint8_t*)nullptr);
    return check_launch("bg_rmsnorm");
}

// The same norm over an fp32 input (the fp32 residual stream): x fp32 [rows, h] with row stride ldx, out bf16.
int bg_rmsnorm_f32(const float* x, int64_t ldx, const void* w, void* out, int64_t ldo, int64_t rows, int64_t h,
                   float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 256 || h > 4096 || ldx % 8 || ldo % 8) {
        bg_set_error("bg_rmsnorm_f32: hidden size must be a multiple of 256 up to 4096 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    launch_rmsnorm_rows(x, ldx, static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out), ldo, rows, h, eps,
                        static_cast<cudaStream_t>(stream));
    return check_launch("bg_rmsnorm_f32");
}

int bg_rmsnorm_mxfp8(const void* x, int64_t ldx, const void* w, void* out_q, void* out_scales, int64_t rows, int64_t h,
                     float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 128 || h > 8192 || ldx % 8) {
        bg_set_error("bg_rmsnorm_mxfp8: hidden size must be a multiple of 128 up to 8192 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    if (launch_rmsnorm_rows(static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w),
                            (__nv_bfloat16*)nullptr, (int64_t)0, rows, h, eps, static_cast<cudaStream_t>(stream),
                            static_cast<uint8_t*>(out_q), static_cast<uint8_t*>(out_scales)))
        return check_launch("bg_rmsnorm_mxfp8");
    launch_kernel(rmsnorm_kernel, dim3((unsigned)rows), dim3(row_threads(h)), 0, static_cast<cudaStream_t>(stream), 0,
                  static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w),
                  (__nv_bfloat16*)nullptr, (int64_t)0, (int)h, eps, static_cast<uint8_t*>(out_q),
                  static_cast<uint8_t*>(out_scales));
    return check_launch("bg_rmsnorm_mxfp8");
}

int bg_add_rmsnorm(const void* y, const void* w_post, void* resid, const void* w_next, void* normed, int64_t rows,
                   int64_t h, float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 8 || h > 8192) {
        bg_set_error("bg_add_rmsnorm: hidden size must be a multiple of 8 up to 8192 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    if (launch_add_rmsnorm_rows(static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(w_post),
                                static_cast<__nv_bfloat16*>(resid), static_cast<const __nv_bfloat16*>(w_next),
                                static_cast<__nv_bfloat16*>(normed), rows, h, eps, static_cast<cudaStream_t>(stream)))
        return check_launch("bg_add_rmsnorm");
    launch_kernel(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(row_threads(h)), 0, static_cast<cudaStream_t>(stream), 0,
                  static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(w_post),
                  static_cast<__nv_bfloat16*>(resid), static_cast<const __nv_bfloat16*>(w_next),
                  static_cast<__nv_bfloat16*>(normed), (int)h, eps, (uint8_t*)nullptr, (uint8_t*)nullptr);
    return check_launch("bg_add_rmsnorm");
}

// bg_add_rmsnorm over an fp32 residual stream: resid fp32 [rows, h] is updated without rounding
// (resid += rmsnorm(y) * (1 + w_post), all in fp32); normed (bf16) feeds the next GEMM.
int bg_add_rmsnorm_f32(const void* y, const void* w_post, float* resid, const void* w_next, void* normed, int64_t rows,
                       int64_t h, float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 256 || h > 4096) {
        bg_set_error("bg_add_rmsnorm_f32: hidden size must be a multiple of 256 up to 4096 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    launch_add_rmsnorm_rows(static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(w_post), resid,
                            static_cast<const __nv_bfloat16*>(w_next), static_cast<__nv_bfloat16*>(normed), rows, h, eps,
                            static_cast<cudaStream_t>(stream));
    return check_launch("bg_add_rmsnorm_f32");
}

// The same with y in fp32 as well (the unrounded output of bg_gemm_bf16_f32out); h a multiple of 256 up to 3072.
int bg_add_rmsnorm_f32y(const float* y, const void* w_post, float* resid, const void* w_next, void* normed, int64_t rows,
                        int64_t h, float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 256 || h > 3072) {
        bg_set_error("bg_add_rmsnorm_f32y: hidden size must be a multiple of 256 up to 3072 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    launch_add_rmsnorm_rows(y, static_cast<const __nv_bfloat16*>(w_post), resid, static_cast<const __nv_bfloat16*>(w_next),
                            static_cast<__nv_bfloat16*>(normed), rows, h, eps, static_cast<cudaStream_t>(stream));
    return check_launch("bg_add_rmsnorm_f32y");
}

int bg_add_rmsnorm_mxfp8(const void* y, const void* w_post, void* resid, const void* w_next, void* normed_q,
                         void* normed_scales, int64_t rows, int64_t h, float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 128 || h > 8192 || w_next == nullptr) {
        bg_set_error("bg_add_rmsnorm_mxfp8: hidden size must be a multiple of 128 up to 8192 (got %lld)", (long long)h);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    if (launch_add_rmsnorm_rows(static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(w_post),
                                static_cast<__nv_bfloat16*>(resid), static_cast<const __nv_bfloat16*>(w_next),
                                (__nv_bfloat16*)nullptr, rows, h, eps, static_cast<cudaStream_t>(stream),
                                static_cast<uint8_t*>(normed_q), static_cast<uint8_t*>(normed_scales)))
        return check_launch("bg_add_rmsnorm_mxfp8");
    launch_kernel(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(row_threads(h)), 0, static_cast<cudaStream_t>(stream), 0,
                  static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(w_post),
                  static_cast<__nv_bfloat16*>(resid), static_cast<const __nv_bfloat16*>(w_next),
                  (__nv_bfloat16*)nullptr, (int)h, eps, static_cast<uint8_t*>(normed_q),
                  static_cast<uint8_t*>(normed_scales));
    return check_launch("bg_add_rmsnorm_mxfp8");
}

static int qk_norm_rope_launch(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads,
                               const void* q_weight, const void* k_weight, const int32_t* positions,
                               const float* inv_freq, const void* cos_table, const void* sin_table,
                               const float* angle_table, int64_t angle_rows, int64_t tokens, int head_dim, float eps,
                               int rotate, void* stream) {
    if (tokens < 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256) || q_heads < 0 || k_heads < 0) {
        bg_set_error("bg_qk_norm_rope: head_dim must be 64, 128 or 256 (got %d)", head_dim);
        return BG_ERR_SHAPE;
    }
    if (ldq % 8 || ldk % 8) {
        bg_set_error("bg_qk_norm_rope: token strides must be multiples of 8 elements");
        return BG_ERR_ALIGN;
    }
    if (tokens == 0) return BG_OK;
    const int warps = 4;
    const unsigned grid = (unsigned)((tokens + warps - 1) / warps);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto* qp = static_cast<__nv_bfloat16*>(q);
    auto* kp = static_cast<__nv_bfloat16*>(k);
    auto* qw = static_cast<const __nv_bfloat16*>(q_weight);
    auto* kw = static_cast<const __nv_bfloat16*>(k_weight);
    auto* ct = static_cast<const __nv_bfloat16*>(cos_table);
    auto* st = static_cast<const __nv_bfloat16*>(sin_table);
    if (qp == nullptr) q_heads = 0;
    if (head_dim == 64)
        launch_kernel(qk_norm_rope_kernel<64>, dim3(grid), dim3(warps * 32), 0, s, 0, qp, ldq, q_heads, kp, ldk, k_heads, qw, kw, positions,
                                                             inv_freq, ct, st, reinterpret_cast<const float2*>(angle_table), (int)angle_rows, tokens, eps, rotate);
    else if (head_dim == 128)
        launch_kernel(qk_norm_rope_kernel<128>, dim3(grid), dim3(warps * 32), 0, s, 0, qp, ldq, q_heads, kp, ldk, k_heads, qw, kw, positions,
                                                              inv_freq, ct, st, reinterpret_cast<const float2*>(angle_table), (int)angle_rows, tokens, eps, rotate);
    else
        launch_kernel(qk_norm_rope_kernel<256>, dim3(grid), dim3(warps * 32), 0, s, 0, qp, ldq, q_heads, kp, ldk, k_heads, qw, kw, positions,
                                                              inv_freq, ct, st, reinterpret_cast<const float2*>(angle_table), (int)angle_rows, tokens, eps, rotate);
    return check_launch("bg_qk_norm_rope");
}

int bg_qk_norm_rope(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads, const void* q_weight,
                    const void* k_weight, const int32_t* positions, const float* inv_freq, int64_t tokens,
                    int head_dim, float eps, int rotate, void* stream) {
    return qk_norm_rope_launch(q, ldq, q_heads, k, ldk, k_heads, q_weight, k_weight, positions, inv_freq, nullptr,
                               nullptr, nullptr, 0, tokens, head_dim, eps, rotate, stream);
}

// The same operation with the angles read from a table made by bg_rope_table ([rows, head_dim / 2] pairs
// (cos, sin) of position * inv_freq; positions are clamped to the table): bit-identical results.
int bg_qk_norm_rope_cached(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads, const void* q_weight,
                           const void* k_weight, const int32_t* positions, const float* rope_table,
                           int64_t table_rows, int64_t tokens, int head_dim, float eps, void* stream) {
    if (positions == nullptr || rope_table == nullptr || table_rows <= 0 ||
        (reinterpret_cast<uintptr_t>(rope_table) & 7)) {
        bg_set_error("bg_qk_norm_rope_cached: positions and an 8-byte aligned table with at least one row are required");
        return BG_ERR_SHAPE;
    }
    return qk_norm_rope_launch(q, ldq, q_heads, k, ldk, k_heads, q_weight, k_weight, positions, nullptr, nullptr,
                               nullptr, rope_table, table_rows, tokens, head_dim, eps, 1, stream);
}

int bg_qk_norm_rope_table(void* q, int64_t ldq, int q_heads, void* k, int64_t ldk, int k_heads,
                          const void* q_weight, const void* k_weight, const void* cos_table, const void* sin_table,
                          int64_t tokens, int head_dim, float eps, void* stream) {
    if (cos_table == nullptr || sin_table == nullptr) {
        bg_set_error("bg_qk_norm_rope_table: cos and sin tables are required");
        return BG_ERR_SHAPE;
    }
    return qk_norm_rope_launch(q, ldq, q_heads, k, ldk, k_heads, q_weight, k_weight, nullptr, nullptr, cos_table,
                               sin_table, nullptr, 0, tokens, head_dim, eps, 1, stream);
}

int bg_rope_table(float* table, int64_t rows, int head_dim, const float* inv_freq, void* stream) {
    if (rows <= 0 || head_dim <= 0 || head_dim % 2) {
        bg_set_error("bg_rope_table: bad shape");
        return BG_ERR_SHAPE;
    }
    const int64_t n = rows * (head_dim / 2);
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<float2*>(table), rows, head_dim / 2, inv_freq);
    return check_launch("bg_rope_table");
}

int bg_transpose_bf16(const void* src, int64_t lds, void* dst, int64_t ldd, int64_t rows, int64_t cols, void* stream) {
    if (rows < 0 || cols < 0 || lds < cols || ldd < rows) {
        bg_set_error("bg_transpose_bf16: bad shape");
        return BG_ERR_SHAPE;
    }
    if (rows == 0 || cols == 0) return BG_OK;
    dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64));
    transpose_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src), lds, static_cast<__nv_bfloat16*>(dst), ldd, rows, cols);
    return check_launch("bg_transpose_bf16");
}

int bg_geglu_backward(const void* gu, const void* dh, void* dgu, int64_t rows, int64_t inter, void* stream) {
    if (rows < 0 || inter <= 0 || inter % 8) {
        bg_set_error("bg_geglu_backward: the intermediate size must be a multiple of 8");
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    const int64_t groups = rows * inter / 8;
    geglu_backward_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(dgu),
        rows, inter);
    return check_launch("bg_geglu_backward");
}

int bg_embed(const int64_t* ids, const void* table, const void* eoi_embedding, void* out, int64_t rows, int64_t h,
             float scale, int64_t eoi_token, int64_t vocab, void* stream) {
    if (rows < 0 || h <= 0 || h % 8 || h > 8192) {
        bg_set_error("bg_embed: hidden size must be a multiple of 8 up to 8192");
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    launch_kernel(embed_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(row_threads(h)), 0, static_cast<cudaStream_t>(stream), 0,
        ids, static_cast<const __nv_bfloat16*>(table), static_cast<const __nv_bfloat16*>(eoi_embedding),
        static_cast<__nv_bfloat16*>(out), (int)h, scale, eoi_token, vocab);
    return check_launch("bg_embed");
}

// bg_embed into an fp32 residual stream: out fp32 [rows, h] = table[id] * scale, not rounded.
int bg_embed_f32(const int64_t* ids, const void* table, const void* eoi_embedding, float* out, int64_t rows, int64_t h,
                 float scale, int64_t eoi_token, int64_t vocab, void* stream) {
    if (rows < 0 || h <= 0 || h % 8 || h > 8192) {
        bg_set_error("bg_embed_f32: hidden size must be a multiple of 8 up to 8192");
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    launch_kernel(embed_kernel<float>, dim3((unsigned)rows), dim3(row_threads(h)), 0, static_cast<cudaStream_t>(stream), 0,
        ids, static_cast<const __nv_bfloat16*>(table), static_cast<const __nv_bfloat16*>(eoi_embedding), out, (int)h, scale,
        eoi_token, vocab);
    return check_launch("bg_embed_f32");
}

int bg_judgment_head(const void* hidden, int64_t ldh, const int32_t* cand_rows, const int32_t* dec_rows,
                     const void* w, const void* cmat, const void* gmat, float* logits, int64_t candidates, int64_t h,
                     int rank, void* stream) {
    if (candidates < 0 || h <= 0 || h % 8 || rank <= 0 || 2 * h * sizeof(float) > 96 * 1024) {
        bg_set_error("bg_judgment_head: bad shape");
        return BG_ERR_SHAPE;
    }
    if (candidates == 0) return BG_OK;
    const size_t smem = 2 * h * sizeof(float);
    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured && smem > 48 * 1024) {
        cudaFuncSetAttribute(judgment_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        configured = true;
    }
    launch_kernel(judgment_head_kernel, dim3((unsigned)candidates, HEAD_SPLIT), dim3(256), smem, static_cast<cudaStream_t>(stream), 0, 
        static_cast<const __nv_bfloat16*>(hidden), ldh, cand_rows, dec_rows, static_cast<const __nv_bfloat16*>(w),
        static_cast<const __nv_bfloat16*>(cmat), static_cast<const __nv_bfloat16*>(gmat), logits, (int)h, rank);
    return check_launch("bg_judgment_head");
}

int bg_candidate_softmax(const float* logits, const int32_t* offsets, double* probs, int64_t questions,
                         double temperature, void* stream) {
    if (questions < 0 || !(temperature > 0.0)) {
        bg_set_error("bg_candidate_softmax: temperature must be finite and positive");
        return BG_ERR_SHAPE;
    }
    if (questions == 0) return BG_OK;
    launch_kernel(candidate_softmax_kernel, dim3((unsigned)((questions + 127) / 128)), dim3(128), 0, static_cast<cudaStream_t>(stream), 0, 
        logits, offsets, probs, (int)questions, temperature);
    return check_launch("bg_candidate_softmax");
}

}  // extern "C"
