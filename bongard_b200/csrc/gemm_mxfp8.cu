// MXFP8 linear path: E4M3 values with one power-of-two (UE8M0) scale per 32 consecutive K elements,
// the block format Blackwell's tensor cores scale by themselves (the reference's `mxfp8` recipe:
// bongard/te_linear.py:32-39, bongard/fused_mlp.py:21-34 hand it to Transformer Engine's
// MXFP8BlockScaling).
//
//   q = e4m3(sat(x * 2^-e)),  e = ceil(log2(amax_32 / 448))  clamped to [-127, 127],  scale byte = e + 127
//   out[m, n] = sum_k (2^ea[m, k/32] * Aq[m, k]) * (2^ew[n, k/32] * Wq[n, k])
//
// Unlike the 128-block recipe (gemm_fp8.cu), nothing is rescaled outside the tensor core:
// `tcgen05.mma.kind::mxf8f6f4.block_scale` multiplies every 32-deep partial product by the two
// scales it reads from tensor memory, so the whole K loop accumulates into one TMEM accumulator
// at the FP8 rate.
//
// Scale layout.  The MMA wants, per 128 rows and per K = 32 step, one scale byte per row, laid
// out in TMEM as 32 lanes x 4 columns (row r -> lane r % 32, column r / 32), the byte inside
// the 32-bit column selected by the instruction (scale id = K step within a 128-deep block), and
// replicated over the four lane quadrants.  `tcgen05.cp.32x128b.warpx4` produces exactly that from
// 512 contiguous bytes of shared memory, so the scales live in global memory in the same 512-byte
// atoms:  atom (r / 128, k / 128),  byte (r % 32) * 16 + (r % 128) / 32 * 4 + (k / 32) % 4.
// A stage of the TMA ring is A 128 x 128 B, W 256 x 128 B, one scale atom for A and two for W.
#include "common.cuh"

#include <cuda_fp8.h>

namespace {

using namespace bg;

constexpr int BM = 128, BN = 256, BK = 128;      // BK = 128 fp8 bytes = one swizzle row = four scale blocks
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK;                  // 16 + 32 KB
constexpr int SF_ATOM = 512;
constexpr int SF_BYTES = 3 * SF_ATOM;                                 // A atom + two W atoms
constexpr int TILE_BYTES = A_BYTES + B_BYTES;
constexpr int SF_OFFSET = STAGES * TILE_BYTES;
constexpr int BAR_OFFSET = SF_OFFSET + STAGES * SF_BYTES;
constexpr int SMEM_BYTES = BAR_OFFSET + 256 + 1024;
constexpr int THREADS = 320;     // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue (two per TMEM lane quadrant)
constexpr int GROUP_M_NARROW = 4, GROUP_M_WIDE = 64;   // row panels per raster group
constexpr int TMEM_SF = 256;      // scale columns behind the 256-column accumulator: per ring parity A at +0, W at +16

struct MxParams {
    int m, n, k, epilogue;
    int64_t ldo;
    __nv_bfloat16* out;
    const uint8_t* a_sf;    // [ceil(m / 128)][k / 128][512]
    const uint8_t* w_sf;    // [w_rows / 128][k / 128][512]
    uint8_t* out_q;         // GeGLU epilogue only: emit the result as MXFP8 (values [m, n], row stride ldo bytes)
    uint8_t* out_sf;        //   and its scale atoms [ceil(m / 128)][n / 128][512]; null -> bf16 output
    int tiles_m, tiles_n;
    int group_m;            // row panels per raster group
    int32_t* status;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
    int per_group = group_m * tiles_n;
    int group = tile / per_group;
    int first_m = group * group_m;
    int rows = min(group_m, tiles_m - first_m);
    int in_group = tile - group * per_group;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

// 1-D bulk copy global -> shared, completing on an mbarrier (16-byte aligned, size multiple of 16).
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Shared-memory descriptor of a 32 x 16-byte block without swizzle (8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
    d |= (uint64_t)(128 >> 4) << 32;      // stride between 8-row groups
    d |= (uint64_t)1 << 46;               // descriptor version for sm_100
    return d;
}
// 32 lanes x 128 bits from shared memory into tensor memory, replicated over the four lane quadrants.
__device__ __forceinline__ void sf_copy(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
// Block-scaled instruction descriptor: E4M3 x E4M3 -> fp32, UE8M0 scales, scale ids = K step in the 128-block.
__device__ __forceinline__ uint32_t idesc_mx(uint32_t m, uint32_t n, uint32_t sf_id) {
    return (sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf_id << 29);
}
__device__ __forceinline__ void mma_mxfp8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                  const MxParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BAR_OFFSET);
    uint64_t* full = bars;                  // [STAGES]
    uint64_t* empty = bars + STAGES;        // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = bars + 2 * STAGES + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 8);
        mbar_fence_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = p.k / BK;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
                // W rows: plain -> 256 consecutive output columns; GeGLU -> 128 gate rows + 128 up rows
                const int w0 = p.epilogue == 1 ? tn * 128 : tn * BN;
                const int w1 = p.epilogue == 1 ? p.n + tn * 128 : tn * BN + 128;
                const int w_rows = p.epilogue == 1 ? 2 * p.n : p.n;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_parked(&empty[stage], phase ^ 1, ab, 501)) break;
                    uint8_t* sa = smem + stage * TILE_BYTES;
                    uint8_t* sb = sa + A_BYTES;
                    uint8_t* sf = smem + SF_OFFSET + stage * SF_BYTES;
                    mbar_expect_tx(&full[stage], TILE_BYTES + SF_BYTES);
                    tma_load_2d(sa, &map_a, &full[stage], kb * BK, tm * BM);
                    tma_load_2d(sb, &map_w, &full[stage], kb * BK, w0);
                    tma_load_2d(sb + B_BYTES / 2, &map_w, &full[stage], kb * BK, w1);
                    bulk_load(sf, p.a_sf + (int64_t(tm) * kblocks + kb) * SF_ATOM, SF_ATOM, &full[stage]);
                    bulk_load(sf + SF_ATOM, p.w_sf + (int64_t(w0 / 128) * kblocks + kb) * SF_ATOM, SF_ATOM, &full[stage]);
                    // a plain tile whose second half lies beyond n reads zero rows there; any valid atom will do
                    const int a1 = w1 < w_rows ? w1 / 128 : w0 / 128;
                    bulk_load(sf + 2 * SF_ATOM, p.w_sf + (int64_t(a1) * kblocks + kb) * SF_ATOM, SF_ATOM, &full[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t step = 0;          // running K-block count: parity selects the scale columns
            int local = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
                // one accumulator: the previous tile has to be drained before it is overwritten
                if (!mbar_wait(acc_empty, (local & 1) ^ 1, ab, 502)) break;
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++step) {
                    if (!mbar_wait(&full[stage], phase, ab, 503)) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * TILE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
                    const uint32_t sf = smem_u32(smem + SF_OFFSET + stage * SF_BYTES);
                    const uint32_t t_sfa = tmem_base + TMEM_SF + (step & 1) * 32;
                    const uint32_t t_sfb = t_sfa + 16;
                    sf_copy(t_sfa, sf_desc(sf));
                    sf_copy(t_sfb, sf_desc(sf + SF_ATOM));
                    sf_copy(t_sfb + 4, sf_desc(sf + 2 * SF_ATOM));
#pragma unroll
                    for (int kk = 0; kk < BK / 32; ++kk) {
                        uint64_t da = smem_desc_sw128(sa + kk * 32, 16, 1024);
                        uint64_t db = smem_desc_sw128(sb + kk * 32, 16, 1024);
                        mma_mxfp8_ss(tmem_base, da, db, idesc_mx(BM, BN, kk), t_sfa, t_sfb, (kb | kk) != 0);
                    }
                    mma_commit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                mma_commit(acc_full);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        // The accumulator is single-buffered, so the epilogue is exposed: two warps per lane quadrant, each
        // draining half of the columns, halve it.
        const int part = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row_in_tile = part * 32 + lane;
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            if (!mbar_wait(acc_full, local & 1, ab, 504)) break;
            tc_fence_after();
            const int row = tm * BM + row_in_tile;
            const uint32_t taddr = tmem_base + (uint32_t(part * 32) << 16);
            if (p.epilogue == 0) {
                const int col0 = tn * BN;
                __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + col0;
#pragma unroll 1
                for (int c = half * (BN / 2); c < (half + 1) * (BN / 2); c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_wait_ld();
                    if (row < p.m) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (col0 + c + v * 8 < p.n) {
                                uint4 o;
                                o.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                                o.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                                o.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                                o.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                                *reinterpret_cast<uint4*>(dst + c + v * 8) = o;
                            }
                        }
                    }
                }
            } else if (p.out_sf != nullptr) {
                // GeGLU result straight to MXFP8: a row's 128 columns of this tile are four 32-blocks = the four
                // scale bytes of one word of the scale atom (row / 128, tn); this warp writes its half of them.
                // The product is rounded to bf16 first, so the values equal quantising the bf16 output afterwards.
                uint8_t* dst = p.out_q + int64_t(row) * p.ldo + tn * 128;
                uint32_t scale_word = 0;
#pragma unroll 1
                for (int c = half * 64; c < (half + 1) * 64; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + c, g);
                    tmem_ld32(taddr + 128 + c, u);
                    tmem_wait_ld();
                    float h[32];
                    float amax = 0.f;
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        h[e] = __bfloat162float(__float2bfloat16_rn(gelu_tanh(__uint_as_float(g[e])) * __uint_as_float(u[e])));
                        amax = fmaxf(amax, fabsf(h[e]));
                    }
                    const int ex = mx_exponent(amax);
                    const float inv = exp2f(float(-ex));
                    scale_word |= uint32_t(ex + 127) << (8 * ((c >> 5) & 1));
                    if (row < p.m) {
#pragma unroll
                        for (int v = 0; v < 2; ++v) {
                            uint4 o;
                            o.x = e4m3x4(h[v * 16 + 0] * inv, h[v * 16 + 1] * inv, h[v * 16 + 2] * inv, h[v * 16 + 3] * inv);
                            o.y = e4m3x4(h[v * 16 + 4] * inv, h[v * 16 + 5] * inv, h[v * 16 + 6] * inv, h[v * 16 + 7] * inv);
                            o.z = e4m3x4(h[v * 16 + 8] * inv, h[v * 16 + 9] * inv, h[v * 16 + 10] * inv, h[v * 16 + 11] * inv);
                            o.w = e4m3x4(h[v * 16 + 12] * inv, h[v * 16 + 13] * inv, h[v * 16 + 14] * inv, h[v * 16 + 15] * inv);
                            *reinterpret_cast<uint4*>(dst + c + v * 16) = o;
                        }
                    }
                }
                if (row < p.m) {
                    const int64_t atom = int64_t(row >> 7) * (p.n / 128) + tn;
                    // this warp's two 32-blocks are half of the row's scale word
                    *reinterpret_cast<uint16_t*>(p.out_sf + atom * SF_ATOM + (row & 31) * 16 + ((row & 127) >> 5) * 4 +
                                                 half * 2) = uint16_t(scale_word);
                }
            } else {
                const int col0 = tn * 128;
                __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + col0;
#pragma unroll 1
                for (int c = half * 64; c < (half + 1) * 64; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + c, g);
                    tmem_ld32(taddr + 128 + c, u);
                    tmem_wait_ld();
                    if (row < p.m) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            float h[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                h[e] = gelu_tanh(__uint_as_float(g[v * 8 + e])) * __uint_as_float(u[v * 8 + e]);
                            uint4 o;
                            o.x = pack_bf16(h[0], h[1]);
                            o.y = pack_bf16(h[2], h[3]);
                            o.z = pack_bf16(h[4], h[5]);
                            o.w = pack_bf16(h[6], h[7]);
                            *reinterpret_cast<uint4*>(dst + c + v * 8) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (ab.raised()) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// A half-warp (16 lanes x 8 elements, one 16-byte load each) covers 128 consecutive K elements of one row,
// i.e. the four scale bytes that share a 32-bit word of the scale atom; four lanes share a 32-element block.
__global__ void quantize_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q,
                                      int64_t ldq, uint8_t* __restrict__ sf, int64_t rows, int kblocks) {
    const int lane = threadIdx.x & 31, l16 = lane & 15;
    const int64_t unit = (int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
    const int64_t row = unit / kblocks;
    const int kb = int(unit % kblocks);
    const bool active = row < rows;
    float f[8];
    float amax = 0.f;
    if (active) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + row * ldx + kb * 128 + l16 * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
            amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
        }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!active) return;
    const int e = mx_exponent(amax);
    const float inv = exp2f(float(-e));
    uint2 out;
    out.x = e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
    out.y = e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
    *reinterpret_cast<uint2*>(q + row * ldq + kb * 128 + l16 * 8) = out;
    if ((l16 & 3) == 0) {
        const int64_t atom = (row >> 7) * kblocks + kb;
        sf[atom * SF_ATOM + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (l16 >> 2)] = uint8_t(e + 127);
    }
}

int launched(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        bg_set_error("%s: launch: %s", what, cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

}  // namespace

extern "C" {

// Bytes of the scale tensor of a [rows, k] matrix: one 512-byte atom per 128 rows x 128 K elements.
int64_t bg_mxfp8_scale_bytes(int64_t rows, int64_t k) { return ((rows + 127) / 128) * (k / 128) * SF_ATOM; }

int bg_quantize_mxfp8(const void* x, int64_t ldx, void* q, int64_t ldq, void* scales, int64_t rows, int64_t k,
                      void* stream) {
    if (rows < 0 || k <= 0 || k % 128 || ldx % 8 || ldq % 8) {
        bg_set_error("bg_quantize_mxfp8: k must be a multiple of 128 (got %lld)", (long long)k);
        return BG_ERR_SHAPE;
    }
    if (rows == 0) return BG_OK;
    const int kblocks = int(k / 128);
    const int64_t units = rows * kblocks;
    quantize_mxfp8_kernel<<<(unsigned)((units + 15) / 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, static_cast<uint8_t*>(scales), rows,
        kblocks);
    return launched("bg_quantize_mxfp8");
}

static int gemm_mxfp8_launch(const void* aq, int64_t lda, const void* a_scales, const void* wq, int64_t ldw,
                             const void* w_scales, void* out, int64_t ldo, void* out_scales, int64_t m, int64_t n,
                             int64_t k, int epilogue, void* stream);

int bg_gemm_mxfp8(const void* aq, int64_t lda, const void* a_scales, const void* wq, int64_t ldw, const void* w_scales,
                  void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue, void* stream) {
    return gemm_mxfp8_launch(aq, lda, a_scales, wq, ldw, w_scales, out, ldo, nullptr, m, n, k, epilogue, stream);
}

// The gate|up GEMM with the GeGLU epilogue writing MXFP8 (values + scale atoms) for the down projection.
int bg_gemm_mxfp8_geglu_q(const void* aq, int64_t lda, const void* a_scales, const void* wq, int64_t ldw,
                          const void* w_scales, void* out_q, int64_t ldq, void* out_scales, int64_t m, int64_t n,
                          int64_t k, void* stream) {
    if (out_scales == nullptr || ldq % 16 || (reinterpret_cast<uintptr_t>(out_scales) & 15)) {
        bg_set_error("bg_gemm_mxfp8_geglu_q: the output needs a 16-byte aligned scale tensor and a row stride multiple of 16");
        return BG_ERR_ALIGN;
    }
    return gemm_mxfp8_launch(aq, lda, a_scales, wq, ldw, w_scales, out_q, ldq, out_scales, m, n, k, 1, stream);
}

static int gemm_mxfp8_launch(const void* aq, int64_t lda, const void* a_scales, const void* wq, int64_t ldw,
                             const void* w_scales, void* out, int64_t ldo, void* out_scales, int64_t m, int64_t n,
                             int64_t k, int epilogue, void* stream) {
    if (m < 0 || n <= 0 || k <= 0 || (epilogue != 0 && epilogue != 1)) {
        bg_set_error("bg_gemm_mxfp8: bad shape");
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    if (k % 128 || n % 128 || lda % 16 || ldw % 16 || (out_scales == nullptr && ldo % 8)) {
        bg_set_error("bg_gemm_mxfp8: k and n must be multiples of 128 (got k=%lld n=%lld)", (long long)k, (long long)n);
        return BG_ERR_SHAPE;
    }
    if ((reinterpret_cast<uintptr_t>(aq) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(out) |
         reinterpret_cast<uintptr_t>(a_scales) | reinterpret_cast<uintptr_t>(w_scales)) & 15) {
        bg_set_error("bg_gemm_mxfp8: pointers must be 16-byte aligned");
        return BG_ERR_ALIGN;
    }
    const int64_t w_rows = epilogue == 1 ? 2 * n : n;
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)w_rows}, str_w[1] = {(uint64_t)ldw};
    uint32_t box_a[2] = {BK, BM}, box_w[2] = {BK, 128};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, aq, dims_a, str_a, box_a,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, wq, dims_w, str_w, box_w,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;

    MxParams p;
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.epilogue = epilogue; p.ldo = ldo;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.out_q = static_cast<uint8_t*>(out);
    p.out_sf = static_cast<uint8_t*>(out_scales);
    p.a_sf = static_cast<const uint8_t*>(a_scales);
    p.w_sf = static_cast<const uint8_t*>(w_scales);
    p.tiles_m = (int)((m + BM - 1) / BM);
    p.tiles_n = epilogue == 1 ? (int)(n / 128) : (int)((n + BN - 1) / BN);
    // raster: few column panels (down, q|k|v, output projections) -> small groups of row panels; many
    // (gate | up) -> large ones (measured at 32 768 rows: down 1 918 -> 1 962 TFLOP/s with 4 instead of 16)
    p.group_m = p.tiles_n < 32 ? GROUP_M_NARROW : GROUP_M_WIDE;
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;
    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            bg_set_error("bg_gemm_mxfp8: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < bg_num_sms() ? tiles : bg_num_sms();
    gemm_mxfp8_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(map_a, map_w, p);
    return launched("bg_gemm_mxfp8");
}

}  // extern "C"
