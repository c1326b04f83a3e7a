// FP8 E4M3 linear path with per-128 block scales.
//
// Scaling recipe (dynamic, per call, no history - the rule of the reference's FP8 linears,
// bongard/float8_training.py:35-44, at 128-element granularity):
//   activations  one scale per row and 128 consecutive K elements   (1 x 128 blocks)
//   weights      one scale per 128 x 128 tile
//   scale = 448 / max(amax, 1e-12);  q = e4m3(sat(x * scale));  the inverse scale is stored.
//
// GEMM: out[m, n] = sum_kb a_inv[m, kb] * w_inv[n / 128, kb] * (Aq[m, kb] . Wq[n, kb]^T)
// tcgen05 block-scaled MMA only knows 1 x 32 UE8M0 scale vectors, so 128-wide fp32 scales are
// applied outside the tensor core: every 128-deep K block is contracted into a fresh TMEM
// accumulator (4 x tcgen05.mma kind::f8f6f4, M128 N256 K32), and eight promotion warps read it
// back (tcgen05.ld), multiply by the two block scales and accumulate in fp32 registers while
// the tensor core works on the next K block in the other TMEM buffer.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 promotion + epilogue.  A promotion
// warp owns 32 rows (its TMEM lane quarter) and 64 + 64 columns: [64s, 64s+64) of the first
// 128-column half of the tile and the same range of the second half, so that for the GeGLU
// epilogue (first half = gate columns, second half = matching up columns) the product
// gelu_tanh(gate) * up is thread-local.
#include "common.cuh"

#include <cuda_fp8.h>

namespace {

using namespace bg;

constexpr int BM = 128, BN = 256, BK = 128;      // BK bytes = 128 fp8 = one swizzle row = one scale block
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;   // 16 + 32 KB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 320;
constexpr int GROUP_M_NARROW = 4, GROUP_M_WIDE = 64;   // row panels per raster group

struct Fp8Params {
    int m, n, k, epilogue;
    int64_t ldo;
    __nv_bfloat16* out;
    const float* a_inv;     // [k / 128, m]   (K-block major: coalesced per-row reads)
    const float* w_inv;     // [w_rows / 128, k / 128]
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

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const Fp8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* part_full = bars + 2 * STAGES;        // [2]
    uint64_t* part_empty = bars + 2 * STAGES + 2;   // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&part_full[b], 1);
            mbar_init(&part_empty[b], 8);
        }
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
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
                const int w0 = p.epilogue == 1 ? tn * 128 : tn * BN;
                const int w1 = p.epilogue == 1 ? p.n + tn * 128 : tn * BN + 128;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_parked(&empty[stage], phase ^ 1, ab, 301)) break;
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    uint8_t* sb = sa + A_BYTES;
                    mbar_expect_tx(&full[stage], STAGE_BYTES);
                    tma_load_2d(sa, &map_a, &full[stage], kb * BK, tm * BM);
                    tma_load_2d(sb, &map_w, &full[stage], kb * BK, w0);
                    tma_load_2d(sb + B_BYTES / 2, &map_w, &full[stage], kb * BK, w1);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, BN, 0, 0, 0, 0);   // E4M3 x E4M3 -> fp32
            int stage = 0;
            uint32_t phase = 0;
            uint32_t step = 0;      // running K-block count: selects the TMEM partial buffer
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < kblocks; ++kb, ++step) {
                    const int buf = step & 1;
                    if (!mbar_wait(&full[stage], phase, ab, 302)) break;
                    if (!mbar_wait(&part_empty[buf], ((step >> 1) & 1) ^ 1, ab, 303)) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 32; ++kk) {
                        uint64_t da = smem_desc_sw128(sa + kk * 32, 16, 1024);
                        uint64_t db = smem_desc_sw128(sb + kk * 32, 16, 1024);
                        mma_fp8_ss(tmem_base + buf * BN, da, db, idesc, kk != 0);
                    }
                    mma_commit(&empty[stage]);
                    mma_commit(&part_full[buf]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else {
        const int part = warp & 3;                 // TMEM lane quarter
        const int slice = (warp - 2) >> 2;         // which 64-column slice of each 128-column half
        const int row_in_tile = part * 32 + lane;
        const uint32_t lane_addr = uint32_t(part * 32) << 16;
        const int kb_stride = p.k / BK;
        uint32_t step = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            const int row = tm * BM + row_in_tile;
            const int safe_row = row < p.m ? row : p.m - 1;
            // weight scale rows of the two 128-column halves of this tile
            const int nb0 = p.epilogue == 1 ? tn : tn * 2;
            const int nb1 = p.epilogue == 1 ? p.n / 128 + tn : tn * 2 + 1;
            const int w_blocks = p.epilogue == 1 ? 2 * p.n / 128 : (p.n + 127) / 128;
            const float* w0 = p.w_inv + int64_t(nb0) * kb_stride;
            const float* w1 = p.w_inv + int64_t(nb1 < w_blocks ? nb1 : nb0) * kb_stride;
            uint64_t acc2[64];                      // 128 fp32 accumulators as packed pairs
#pragma unroll
            for (int i = 0; i < 64; ++i) acc2[i] = 0ull;
            for (int kb = 0; kb < kblocks; ++kb, ++step) {
                const int buf = step & 1;
                const float sa = p.a_inv[int64_t(kb) * p.m + safe_row];
                const float s0 = sa * w0[kb], s1 = sa * w1[kb];
                if (!mbar_wait(&part_full[buf], (step >> 1) & 1, ab, 304)) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + lane_addr + buf * BN + slice * 64;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld32(taddr + (c >> 1) * 128 + (c & 1) * 32, r);
                    tmem_wait_ld();
                    const float s = (c >> 1) ? s1 : s0;
                    const uint64_t s2 = pack_f32x2(s, s);
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        acc2[c * 16 + i] = fma_f32x2(pack_u32x2(r[2 * i], r[2 * i + 1]), s2, acc2[c * 16 + i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&part_empty[buf]);
            }
            const float* acc = reinterpret_cast<const float*>(acc2);
            if (row < p.m) {
                if (p.epilogue == 0) {
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int col0 = tn * BN + h2 * 128 + slice * 64;
                        __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + col0;
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            if (col0 + v * 8 < p.n) {
                                const float* a = acc + h2 * 64 + v * 8;
                                uint4 o;
                                o.x = pack_bf16(a[0], a[1]);
                                o.y = pack_bf16(a[2], a[3]);
                                o.z = pack_bf16(a[4], a[5]);
                                o.w = pack_bf16(a[6], a[7]);
                                *reinterpret_cast<uint4*>(dst + v * 8) = o;
                            }
                        }
                    }
                } else {
                    const int col0 = tn * 128 + slice * 64;
                    __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + col0;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float h[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) h[e] = gelu_tanh(acc[v * 8 + e]) * acc[64 + v * 8 + e];
                        uint4 o;
                        o.x = pack_bf16(h[0], h[1]);
                        o.y = pack_bf16(h[2], h[3]);
                        o.z = pack_bf16(h[4], h[5]);
                        o.w = pack_bf16(h[6], h[7]);
                        *reinterpret_cast<uint4*>(dst + v * 8) = o;
                    }
                }
            }
        }
    }

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

// ---------------------------------------------------------------------------- quantisation

// 1 x 128 blocks: a half-warp per block (16 lanes x 8 elements), two blocks per warp.
__global__ void quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q,
                                     int64_t ldq, float* __restrict__ inv_t, int64_t m, int kblocks) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
    const int64_t row = unit / kblocks;
    const int kb = int(unit % kblocks);
    const bool active = row < m;
    float f[8];
    float amax = 0.f;
    if (active) {
        const uint4 v = *reinterpret_cast<const uint4*>(x + row * ldx + kb * 128 + (lane & 15) * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
            amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
        }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!active) return;
    const float scale = 448.f / fmaxf(amax, 1e-12f);
    uint2 out;
    out.x = e4m3x4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
    out.y = e4m3x4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
    *reinterpret_cast<uint2*>(q + row * ldq + kb * 128 + (lane & 15) * 8) = out;
    if ((lane & 15) == 0) inv_t[int64_t(kb) * m + row] = 1.f / scale;
}

// 128 x 128 tiles: one block of 256 threads per tile (weights, quantised once at load time).
__global__ void quantize_tiles_kernel(const __nv_bfloat16* __restrict__ w, int64_t ldw, uint8_t* __restrict__ q,
                                      int64_t ldq, float* __restrict__ inv, int64_t n, int kblocks) {
    __shared__ float red[8];
    const int kb = blockIdx.x, nb = blockIdx.y;
    const int r0 = threadIdx.x >> 4, c = (threadIdx.x & 15) * 8;     // 16 rows x 16 chunks per pass
    float amax = 0.f;
    for (int r = r0; r < 128; r += 16) {
        const int64_t row = int64_t(nb) * 128 + r;
        if (row < n) {
            const uint4 v = *reinterpret_cast<const uint4*>(w + row * ldw + kb * 128 + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 t = __bfloat1622float2(h[i]);
                amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
            }
        }
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    const float scale = 448.f / fmaxf(amax, 1e-12f);
    for (int r = r0; r < 128; r += 16) {
        const int64_t row = int64_t(nb) * 128 + r;
        if (row < n) {
            const uint4 v = *reinterpret_cast<const uint4*>(w + row * ldw + kb * 128 + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            float f[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 t = __bfloat1622float2(h[i]);
                f[2 * i] = t.x * scale;
                f[2 * i + 1] = t.y * scale;
            }
            uint2 out;
            out.x = e4m3x4(f[0], f[1], f[2], f[3]);
            out.y = e4m3x4(f[4], f[5], f[6], f[7]);
            *reinterpret_cast<uint2*>(q + row * ldq + kb * 128 + c) = out;
        }
    }
    if (threadIdx.x == 0) inv[int64_t(nb) * kblocks + kb] = 1.f / scale;
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

int bg_quantize_e4m3_rows(const void* x, int64_t ldx, void* q, int64_t ldq, float* inv_scale_t, int64_t m, int64_t k,
                          void* stream) {
    if (m < 0 || k <= 0 || k % 128 || ldx % 8 || ldq % 16) {
        bg_set_error("bg_quantize_e4m3_rows: k must be a multiple of 128 (got %lld); ldx %% 8 == 0, ldq %% 16 == 0",
                     (long long)k);
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    const int kblocks = int(k / 128);
    const int64_t units = m * kblocks;              // half-warps
    const int warps = 8;
    const unsigned grid = (unsigned)((units + 2 * warps - 1) / (2 * warps));
    quantize_rows_kernel<<<grid, warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, inv_scale_t, m, kblocks);
    return launched("bg_quantize_e4m3_rows");
}

int bg_quantize_e4m3_tiles(const void* w, int64_t ldw, void* q, int64_t ldq, float* inv_scale, int64_t n, int64_t k,
                           void* stream) {
    if (n <= 0 || k <= 0 || k % 128 || ldw % 8 || ldq % 16) {
        bg_set_error("bg_quantize_e4m3_tiles: k must be a multiple of 128 (got %lld)", (long long)k);
        return BG_ERR_SHAPE;
    }
    dim3 grid((unsigned)(k / 128), (unsigned)((n + 127) / 128));
    quantize_tiles_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(w), ldw, static_cast<uint8_t*>(q), ldq, inv_scale, n, int(k / 128));
    return launched("bg_quantize_e4m3_tiles");
}

int bg_gemm_fp8_block128(const void* aq, int64_t lda, const float* a_inv_t, const void* wq, int64_t ldw,
                         const float* w_inv, void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue,
                         void* stream) {
    if (m < 0 || n <= 0 || k <= 0 || (epilogue != 0 && epilogue != 1)) {
        bg_set_error("bg_gemm_fp8_block128: bad shape");
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    if (k % 128 || n % 128 || lda % 16 || ldw % 16 || ldo % 8) {
        bg_set_error("bg_gemm_fp8_block128: k and n must be multiples of 128 (got k=%lld n=%lld)", (long long)k,
                     (long long)n);
        return BG_ERR_ALIGN;
    }
    if ((reinterpret_cast<uintptr_t>(aq) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(out)) & 15) {
        bg_set_error("bg_gemm_fp8_block128: pointers must be 16-byte aligned");
        return BG_ERR_ALIGN;
    }
    const int64_t w_rows = epilogue == 1 ? 2 * n : n;
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)w_rows}, str_w[1] = {(uint64_t)ldw};
    uint32_t box[2] = {BK, 128};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, aq, dims_a, str_a, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, wq, dims_w, str_w, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    Fp8Params p;
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.epilogue = epilogue; p.ldo = ldo;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.a_inv = a_inv_t; p.w_inv = w_inv;
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
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            bg_set_error("bg_gemm_fp8_block128: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < bg_num_sms() ? tiles : bg_num_sms();
    gemm_fp8_kernel<<<grid, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(map_a, map_w, p);
    return launched("bg_gemm_fp8_block128");
}

// Scratch needed by bg_linear_fp8 for an [m, k] activation: the quantised copy (rows padded to
// 16 bytes) followed by the fp32 inverse scales [k / 128, m].
int64_t bg_linear_fp8_workspace_bytes(int64_t m, int64_t k) {
    const int64_t q = ((m * k + 255) / 256) * 256;
    return q + (k / 128) * m * 4;
}

// x (bf16) is quantised into the caller's workspace, then contracted with pre-quantised weights.
int bg_linear_fp8(const void* x, int64_t ldx, const void* wq, int64_t ldw, const float* w_inv, void* out,
                  int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue, void* workspace,
                  int64_t workspace_bytes, void* stream) {
    if (m == 0) return BG_OK;
    if (k <= 0 || k % 128) {
        bg_set_error("bg_linear_fp8: k must be a multiple of 128 (got %lld)", (long long)k);
        return BG_ERR_ALIGN;
    }
    if (workspace == nullptr || workspace_bytes < bg_linear_fp8_workspace_bytes(m, k) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255)) {
        bg_set_error("bg_linear_fp8: workspace of %lld bytes (256-byte aligned) required",
                     (long long)bg_linear_fp8_workspace_bytes(m, k));
        return BG_ERR_WORKSPACE;
    }
    uint8_t* q = static_cast<uint8_t*>(workspace);
    float* inv = reinterpret_cast<float*>(q + ((m * k + 255) / 256) * 256);
    int rc = bg_quantize_e4m3_rows(x, ldx, q, k, inv, m, k, stream);
    if (rc) return rc;
    return bg_gemm_fp8_block128(q, k, inv, wq, ldw, w_inv, out, ldo, m, n, k, epilogue, stream);
}

// ---------------------------------------------------------------------------- allocation-free variant
//
// Some callers are not in a position to hand over scratch memory: a plugin invoked by a host
// runtime that has already reserved the device's memory for its own pools, a callback that runs
// where calling into the allocator is forbidden or would stall the device, an integration that
// simply has no allocator of its own.  For them the scratch of the FP8 linear lives inside the
// library, in a fixed file-scope device array.  Every GPU that loads the library carries these
// BG_FP8_STATIC_SCRATCH_BYTES until the process exits, so the limit is kept modest.
//
// The array's name is only a host-side handle: the kernels need its device address, which is
// looked up once per device (with that device current) by cudaGetSymbolAddress on the first call
// there.  Do that first call before starting any stream capture.
//
// All calls on a device share the one array and it keeps whatever the last call left in it.
// Nothing in it has to start at zero (each call overwrites exactly the part it then reads), but
// two calls whose kernels overlap on the GPU - different streams, no ordering between them -
// would overwrite each other's quantised activations: order them on one stream or with events.
constexpr int64_t kStaticScratchBytes = 9ll << 20;     // 8 Mi activation elements + their block scales
constexpr int kMaxDevices = kBgMaxDevices;
static __device__ __align__(256) uint8_t g_fp8_static_scratch[kStaticScratchBytes];

int64_t bg_linear_fp8_static_max_bytes(void) { return kStaticScratchBytes; }

int bg_linear_fp8_static(const void* x, int64_t ldx, const void* wq, int64_t ldw, const float* w_inv, void* out,
                         int64_t ldo, int64_t m, int64_t n, int64_t k, int epilogue, void* stream) {
    if (m == 0) return BG_OK;
    if (m < 0 || k <= 0 || k % 128) {
        bg_set_error("bg_linear_fp8_static: k must be a positive multiple of 128 (got %lld)", (long long)k);
        return BG_ERR_ALIGN;
    }
    const int64_t need = bg_linear_fp8_workspace_bytes(m, k);
    if (need > kStaticScratchBytes) {
        bg_set_error("bg_linear_fp8_static: an activation of %lld x %lld needs %lld bytes of scratch, the built-in "
                     "buffer holds %lld; split the rows or use bg_linear_fp8 with a caller-owned workspace",
                     (long long)m, (long long)k, (long long)need, (long long)kStaticScratchBytes);
        return BG_ERR_WORKSPACE;
    }
    static void* device_address[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        bg_set_error("bg_linear_fp8_static: cannot identify the current device (%s)", cudaGetErrorString(e));
        return BG_ERR_DRIVER;
    }
    if (device_address[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_fp8_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            bg_set_error("bg_linear_fp8_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return BG_ERR_DRIVER;
        }
        device_address[dev] = ptr;
    }
    uint8_t* q = static_cast<uint8_t*>(device_address[dev]);
    float* inv = reinterpret_cast<float*>(q + ((m * k + 255) / 256) * 256);
    int rc = bg_quantize_e4m3_rows(x, ldx, q, k, inv, m, k, stream);
    if (rc) return rc;
    return bg_gemm_fp8_block128(q, k, inv, wq, ldw, w_inv, out, ldo, m, n, k, epilogue, stream);
}

}  // extern "C"
