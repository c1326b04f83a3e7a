// Backward of the memory-bound glue: RMSNorm with the zero-centred gain, and QK-norm + rotary
// embedding.  Both are one pass over the rows (input, upstream gradient in; input gradient out) with
// the gain gradient accumulated per thread in registers over the rows a block (or warp) walks,
// written as one partial row per block (warp) and summed in a fixed order by a second kernel:
// no atomics, so results do not depend on scheduling.  HBM bandwidth bounds them.
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

// Block-wide sums of two values at once; every thread receives both totals.  `scratch` holds 66 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();   // scratch may still be read from the previous row
    if (lane == 0) {
        scratch[warp] = a;
        scratch[33 + warp] = b;
    }
    __syncthreads();
    const float ta = lane < warps ? scratch[lane] : 0.f;
    const float tb = lane < warps ? scratch[33 + lane] : 0.f;
    return make_float2(warp_sum(ta), warp_sum(tb));
}

// y = x * r * (1 + w), r = rsqrt(mean(x^2) + eps)   (transformers modeling_t5gemma2.py:61-69, fp32 math)
//   g  = dy * (1 + w)
//   dx = r * g - x * r^3 * mean(g * x)
//   dw = sum over rows of dy * x * r
// Block b walks rows b, b + gridDim.x, ...; thread t owns columns 8t .. 8t+7 of every row.
__global__ void rmsnorm_backward_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                        const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                                        int64_t lddy, __nv_bfloat16* __restrict__ dx, int64_t lddx,
                                        float* __restrict__ partial, int64_t rows, int h, float eps) {
    __shared__ float scratch[66];
    const int c = threadIdx.x * 8;
    const bool active = c < h;
    float gain[8], dw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) gain[i] = dw[i] = 0.f;
    if (active) {
        unpack8(*reinterpret_cast<const uint4*>(w + c), gain);
#pragma unroll
        for (int i = 0; i < 8; ++i) gain[i] += 1.f;
    }
    // the loads of the next row are issued before this row's reduction, so two rows are in flight per block
    uint4 raw_x = make_uint4(0, 0, 0, 0), raw_d = make_uint4(0, 0, 0, 0);
    if (active && int64_t(blockIdx.x) < rows) {
        raw_x = *reinterpret_cast<const uint4*>(x + int64_t(blockIdx.x) * ldx + c);
        raw_d = __ldcs(reinterpret_cast<const uint4*>(dy + int64_t(blockIdx.x) * lddy + c));
    }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float xv[8], g[8];
        float ss = 0.f, dot = 0.f;
        unpack8(raw_x, xv);
        unpack8(raw_d, g);
        const int64_t next = row + gridDim.x;
        if (active && next < rows) {
            raw_x = *reinterpret_cast<const uint4*>(x + next * ldx + c);
            raw_d = __ldcs(reinterpret_cast<const uint4*>(dy + next * lddy + c));
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ss += xv[i] * xv[i];
            dot += g[i] * gain[i] * xv[i];
        }
        const float2 t = block_sum2(ss, dot, scratch);
        const float r = rsqrtf(t.x / float(h) + eps);
        const float k = r * r * r * t.y / float(h);
        if (active) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dw[i] += g[i] * xv[i] * r;
                o[i] = r * g[i] * gain[i] - xv[i] * k;
            }
            *reinterpret_cast<uint4*>(dx + row * lddx + c) = pack8(o);
        }
    }
    if (active) {
        float* dst = partial + int64_t(blockIdx.x) * h + c;
        *reinterpret_cast<float4*>(dst) = make_float4(dw[0], dw[1], dw[2], dw[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(dw[4], dw[5], dw[6], dw[7]);
    }
}

// h = gelu_tanh(g) * u for gu = [g | u] ([rows, 2 inter] bf16): the activation as its own pass, for the training
// forward that keeps gu for the backward instead of recomputing it (transformers modeling_t5gemma2.py:87-91
// computes it from the bf16 projections the same way).
__global__ void geglu_forward_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, int64_t rows,
                                     int64_t inter) {
    const int64_t i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i >= rows * inter) return;
    const int64_t row = i / inter, col = i % inter;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + row * 2 * inter + col), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter + col), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gelu_tanh(g[e]) * u[e];
    *reinterpret_cast<uint4*>(h + i) = pack8(o);
}

// Sum of the partial rows, columns below `split` to out0 and the others to out1.  A block owns 32 columns: its
// eight warps each add every eighth row (128-byte coalesced reads), then the eight sums are added in warp order,
// so the result does not depend on scheduling.
__global__ void column_sum_kernel(const float* __restrict__ partial, int64_t parts, int64_t cols, int64_t split,
                                  float* __restrict__ out0, float* __restrict__ out1) {
    __shared__ float sums[8][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t c = int64_t(blockIdx.x) * 32 + lane;
    float acc = 0.f;
    if (c < cols)
        for (int64_t p = warp; p < parts; p += 8) acc += partial[p * cols + c];
    sums[warp][lane] = acc;
    __syncthreads();
    if (warp != 0 || c >= cols) return;
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += sums[w][lane];
    if (c < split) out0[c] = total;
    else if (out1 != nullptr) out1[c - split] = total;
}

// E consecutive bf16 values as 32-bit words (kept in registers: unpacked with shifts, packed with cvt).
template <int E>
struct alignas(2 * E) Raw {
    uint32_t w[E / 2];
};
constexpr int HB = 4;     // heads whose loads are issued together

// Backward of QK-norm + RoPE (forward: bongard/attention.py:172-180, fused form bongard/qk_norm_rope.metal:4-33).
// Forward per head: a = x * r * (1 + w);  y[i] = a[i] cos[i] + sign(i) a[partner(i)] sin[i], sign = -1 for
// i < D/2, partner(i) = (i + D/2) mod D.  Backward:
//   da[j] = dy[j] cos[j] - sign(j) * (dy sin)[partner(j)];   then the RMSNorm backward over the head.
// One warp walks tokens warp_id, warp_id + n_warps, ...; lane l owns elements [l*D/32, (l+1)*D/32) and its
// partner lives in lane l ^ 16.  x is the input the forward normalised (the forward itself runs in place, so
// the caller keeps a copy).  Gain gradients: one partial row of 2*D floats (query gain | key gain) per warp.
template <int D>
__global__ void __launch_bounds__(256, 2) qk_norm_rope_backward_kernel(const __nv_bfloat16* __restrict__ xq, int64_t ldxq,
                                             const __nv_bfloat16* __restrict__ dyq, int64_t lddyq,
                                             __nv_bfloat16* __restrict__ dxq, int64_t lddxq, int q_heads,
                                             const __nv_bfloat16* __restrict__ xk, int64_t ldxk,
                                             const __nv_bfloat16* __restrict__ dyk, int64_t lddyk,
                                             __nv_bfloat16* __restrict__ dxk, int64_t lddxk, int k_heads,
                                             const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                                             const int32_t* __restrict__ positions, const float* __restrict__ inv_freq,
                                             const __nv_bfloat16* __restrict__ cos_table,
                                             const __nv_bfloat16* __restrict__ sin_table, float* __restrict__ partial,
                                             int64_t tokens, float eps, int rotate) {
    constexpr int E = D / 32;
    const int lane = threadIdx.x & 31;
    const int64_t warp_id = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t n_warps = int64_t(gridDim.x) * (blockDim.x >> 5);
    float gq[E], gk[E], dwq[E], dwk[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        gq[e] = 1.f + __bfloat162float(qw[lane * E + e]);
        gk[e] = xk != nullptr ? 1.f + __bfloat162float(kw[lane * E + e]) : 0.f;
        dwq[e] = dwk[e] = 0.f;
    }
    const float sign = lane < 16 ? -1.f : 1.f;
    for (int64_t token = warp_id; token < tokens; token += n_warps) {
        float cs[E], sn[E];
        if (rotate && cos_table != nullptr) {
#pragma unroll
            for (int e = 0; e < E; ++e) {
                cs[e] = __bfloat162float(cos_table[token * D + lane * E + e]);
                sn[e] = __bfloat162float(sin_table[token * D + lane * E + e]);
            }
        } else if (rotate) {
            const float pos = float(positions[token]);
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const int i = (lane * E + e) & (D / 2 - 1);
                sincosf(pos * inv_freq[i], &sn[e], &cs[e]);
            }
        }
        // heads in batches of HB: all loads of a batch are issued before the first reduction
        const int heads = q_heads + (xk != nullptr ? k_heads : 0);
        for (int h0 = 0; h0 < heads; h0 += HB) {
            Raw<E> rx[HB], rd[HB];
#pragma unroll
            for (int b = 0; b < HB; ++b) {
                const int head = h0 + b;
                if (head < heads) {
                    const bool is_q = head < q_heads;
                    const int hh = is_q ? head : head - q_heads;
                    rx[b] = *reinterpret_cast<const Raw<E>*>((is_q ? xq + token * ldxq : xk + token * ldxk) + hh * D + lane * E);
                    rd[b] = *reinterpret_cast<const Raw<E>*>((is_q ? dyq + token * lddyq : dyk + token * lddyk) + hh * D + lane * E);
                }
            }
#pragma unroll
            for (int b = 0; b < HB; ++b) {
                const int head = h0 + b;
                if (head >= heads) continue;
                const bool is_q = head < q_heads;
                const int hh = is_q ? head : head - q_heads;
                __nv_bfloat16* po = (is_q ? dxq + token * lddxq : dxk + token * lddxk) + hh * D + lane * E;
                float xv[E], d[E];
#pragma unroll
                for (int e = 0; e < E; e += 2) {
                    xv[e] = __uint_as_float(rx[b].w[e / 2] << 16);
                    xv[e + 1] = __uint_as_float(rx[b].w[e / 2] & 0xffff0000u);
                    d[e] = __uint_as_float(rd[b].w[e / 2] << 16);
                    d[e + 1] = __uint_as_float(rd[b].w[e / 2] & 0xffff0000u);
                }
                if (rotate) {
#pragma unroll
                    for (int e = 0; e < E; ++e) {
                        const float other = __shfl_xor_sync(0xffffffffu, d[e] * sn[e], 16);
                        d[e] = d[e] * cs[e] - sign * other;
                    }
                }
                float ss = 0.f, dot = 0.f;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float gain = is_q ? gq[e] : gk[e];
                    ss += xv[e] * xv[e];
                    dot += d[e] * gain * xv[e];
                }
                ss = warp_sum(ss);
                dot = warp_sum(dot);
                const float r = rsqrtf(ss / float(D) + eps);
                const float k = r * r * r * dot / float(D);
                float of[E];
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const float gain = is_q ? gq[e] : gk[e];
                    if (is_q) dwq[e] += d[e] * xv[e] * r;
                    else dwk[e] += d[e] * xv[e] * r;
                    of[e] = r * d[e] * gain - xv[e] * k;
                }
                Raw<E> o;
#pragma unroll
                for (int e = 0; e < E; e += 2) o.w[e / 2] = pack_bf16(of[e], of[e + 1]);
                *reinterpret_cast<Raw<E>*>(po) = o;
            }
        }
    }
    float* dst = partial + warp_id * (2 * D) + lane * E;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        dst[e] = dwq[e];
        dst[D + e] = dwk[e];
    }
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        bg_set_error("%s: launch: %s", what, cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

// Grids are one wave: resident blocks per SM (from the occupancy calculator) times the SM count.
int64_t norm_blocks(int64_t rows, int64_t h) {
    const int threads = int(((h / 8) + 31) / 32 * 32);
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rmsnorm_backward_kernel, threads, 0) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    const int64_t cap = int64_t(bg_num_sms()) * per_sm;
    return rows < cap ? rows : cap;
}

constexpr int QK_WARPS = 8;
int64_t qk_blocks(int64_t tokens, int head_dim) {
    int per_sm = 0;
    cudaError_t e = head_dim == 64    ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qk_norm_rope_backward_kernel<64>, QK_WARPS * 32, 0)
                    : head_dim == 128 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qk_norm_rope_backward_kernel<128>, QK_WARPS * 32, 0)
                                      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qk_norm_rope_backward_kernel<256>, QK_WARPS * 32, 0);
    if (e != cudaSuccess || per_sm < 1) per_sm = 1;
    const int64_t need = (tokens + QK_WARPS - 1) / QK_WARPS;
    const int64_t cap = int64_t(bg_num_sms()) * per_sm;
    return need < cap ? need : cap;
}

}  // namespace

extern "C" {

int bg_geglu_forward(const void* gu, void* h, int64_t rows, int64_t inter, void* stream) {
    if (rows < 0 || inter <= 0 || inter % 8) {
        bg_set_error("bg_geglu_forward: the intermediate size must be a multiple of 8");
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    const int64_t groups = rows * inter / 8;
    geglu_forward_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), rows, inter);
    return check_launch("bg_geglu_forward");
}

int64_t bg_rmsnorm_backward_workspace_bytes(int64_t rows, int64_t h) {
    return rows <= 0 ? 0 : norm_blocks(rows, h) * h * int64_t(sizeof(float));
}

int bg_rmsnorm_backward(const void* x, int64_t ldx, const void* w, const void* dy, int64_t lddy, void* dx,
                        int64_t lddx, float* dw, void* workspace, int64_t workspace_bytes, int64_t rows, int64_t h,
                        float eps, void* stream) {
    if (rows < 0 || h <= 0 || h % 8 || h > 8192 || ldx < h || lddy < h || lddx < h || ldx % 8 || lddy % 8 || lddx % 8) {
        bg_set_error("bg_rmsnorm_backward: the width must be a multiple of 8 up to 8192 and the row strides multiples of 8");
        return BG_ERR_SHAPE;
    }
    if (workspace_bytes < bg_rmsnorm_backward_workspace_bytes(rows, h) || (rows > 0 && workspace == nullptr)) {
        bg_set_error("bg_rmsnorm_backward: the workspace is too small");
        return BG_ERR_WORKSPACE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        cudaMemsetAsync(dw, 0, h * sizeof(float), s);
        return check_launch("bg_rmsnorm_backward");
    }
    const int64_t blocks = norm_blocks(rows, h);
    const int threads = int(((h / 8) + 31) / 32 * 32);
    rmsnorm_backward_kernel<<<(unsigned)blocks, threads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(w),
        static_cast<const __nv_bfloat16*>(dy), lddy, static_cast<__nv_bfloat16*>(dx), lddx,
        static_cast<float*>(workspace), rows, int(h), eps);
    column_sum_kernel<<<(unsigned)((h + 31) / 32), 256, 0, s>>>(static_cast<const float*>(workspace), blocks, h, h, dw,
                                                                  nullptr);
    return check_launch("bg_rmsnorm_backward");
}

int64_t bg_qk_norm_rope_backward_workspace_bytes(int64_t tokens, int head_dim) {
    return tokens <= 0 ? 0 : qk_blocks(tokens, head_dim) * QK_WARPS * 2 * head_dim * int64_t(sizeof(float));
}

int bg_qk_norm_rope_backward(const void* xq, int64_t ldxq, const void* dyq, int64_t lddyq, void* dxq, int64_t lddxq,
                             int q_heads, const void* xk, int64_t ldxk, const void* dyk, int64_t lddyk, void* dxk,
                             int64_t lddxk, int k_heads, const void* q_weight, const void* k_weight,
                             const int32_t* positions, const float* inv_freq, const void* cos_table,
                             const void* sin_table, float* dq_weight, float* dk_weight, void* workspace,
                             int64_t workspace_bytes, int64_t tokens, int head_dim, float eps, int rotate,
                             void* stream) {
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) {
        bg_set_error("bg_qk_norm_rope_backward: head_dim must be 64, 128 or 256");
        return BG_ERR_SHAPE;
    }
    const bool tables = cos_table != nullptr && sin_table != nullptr;
    if (tokens < 0 || q_heads <= 0 || k_heads < 0 || (rotate && !tables && (positions == nullptr || inv_freq == nullptr)) ||
        ((ldxq | lddyq | lddxq | ldxk | lddyk | lddxk) % 8)) {
        bg_set_error("bg_qk_norm_rope_backward: bad shape (strides must be multiples of 8; rotation needs positions and "
                     "inverse frequencies, or cos and sin tables)");
        return BG_ERR_SHAPE;
    }
    if (workspace_bytes < bg_qk_norm_rope_backward_workspace_bytes(tokens, head_dim) ||
        (tokens > 0 && workspace == nullptr)) {
        bg_set_error("bg_qk_norm_rope_backward: the workspace is too small");
        return BG_ERR_WORKSPACE;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (tokens == 0) {
        cudaMemsetAsync(dq_weight, 0, head_dim * sizeof(float), s);
        if (dk_weight != nullptr) cudaMemsetAsync(dk_weight, 0, head_dim * sizeof(float), s);
        return check_launch("bg_qk_norm_rope_backward");
    }
    const int64_t blocks = qk_blocks(tokens, head_dim);
    if (k_heads == 0) xk = nullptr;
    auto launch = [&](auto kernel) {
        kernel<<<(unsigned)blocks, QK_WARPS * 32, 0, s>>>(
            static_cast<const __nv_bfloat16*>(xq), ldxq, static_cast<const __nv_bfloat16*>(dyq), lddyq,
            static_cast<__nv_bfloat16*>(dxq), lddxq, q_heads, static_cast<const __nv_bfloat16*>(xk), ldxk,
            static_cast<const __nv_bfloat16*>(dyk), lddyk, static_cast<__nv_bfloat16*>(dxk), lddxk, k_heads,
            static_cast<const __nv_bfloat16*>(q_weight), static_cast<const __nv_bfloat16*>(k_weight), positions,
            inv_freq, tables ? static_cast<const __nv_bfloat16*>(cos_table) : nullptr,
            tables ? static_cast<const __nv_bfloat16*>(sin_table) : nullptr, static_cast<float*>(workspace), tokens, eps,
            rotate);
    };
    if (head_dim == 64) launch(qk_norm_rope_backward_kernel<64>);
    else if (head_dim == 128) launch(qk_norm_rope_backward_kernel<128>);
    else launch(qk_norm_rope_backward_kernel<256>);
    // the partial rows are [query gain | key gain]
    column_sum_kernel<<<(unsigned)((2 * head_dim + 31) / 32), 256, 0, s>>>(
        static_cast<const float*>(workspace), blocks * QK_WARPS, 2 * head_dim, head_dim, dq_weight, dk_weight);
    return check_launch("bg_qk_norm_rope_backward");
}

}  // extern "C"
