// BF16 projection / MLP contraction on the 5th-generation tensor cores.
//
//   out[M, N] = A[M, K] . W[N, K]^T          (both operands K-contiguous: x @ W.T of F.linear)
//
// One persistent CTA per SM walks output tiles of 128 x 256.  Warp 0 streams A and W tiles
// into a 4-stage shared-memory ring with TMA (128-byte swizzle); warp 1 issues
// tcgen05.mma (M128 N256 K16) into one of two 256-column TMEM accumulators; warps 2-5 drain
// the other accumulator (tcgen05.ld), apply the epilogue and store bf16, so the epilogue of
// tile i overlaps the main loop of tile i+1.
//
// Epilogues:
//   0  plain        out = acc
//   1  GeGLU        W is the stacked [gate; up] weight of 2N rows; each CTA tile holds 128 gate
//                   columns and the matching 128 up columns, and stores gelu_tanh(gate) * up.
//                   This is the fused gate_up GEMM + activation of the reference's TEMLP
//                   (bongard/te_linear.py:98-103) without ever writing gate/up to memory.
#include "common.cuh"

namespace {

using namespace bg;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;            // 64 bf16 = one 128-byte swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int B_BYTES = BN * BK * 2;        // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int THREADS = 192;

struct GemmParams {
    int m, n, k;                  // n = output columns
    int epilogue;
    int64_t ldo;
    __nv_bfloat16* out;
    int tiles_m, tiles_n;
    int group_m;                  // raster: this many row-tiles share each weight panel while it is in L2
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
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                 // [STAGES]
    uint64_t* empty = bars + STAGES;       // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;      // [2]
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
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
    pdl_wait();                   // the predecessor in the stream has finished; from here on global memory may be touched
    pdl_launch_dependents();      // the successor may start its own prologue

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = (p.k + BK - 1) / BK;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
                const int row0 = tm * BM;
                // W rows: plain -> 256 consecutive output columns; GeGLU -> 128 gate rows + 128 up rows.
                const int w0 = p.epilogue == 1 ? tn * 128 : tn * BN;
                const int w1 = p.epilogue == 1 ? p.n + tn * 128 : tn * BN + 128;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait_parked(&empty[stage], phase ^ 1, ab, 101)) break;
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    uint8_t* sb = sa + A_BYTES;
                    mbar_expect_tx(&full[stage], STAGE_BYTES);
                    tma_load_2d(sa, &map_a, &full[stage], kb * BK, row0);
                    tma_load_2d(sb, &map_w, &full[stage], kb * BK, w0);
                    tma_load_2d(sb + B_BYTES / 2, &map_w, &full[stage], kb * BK, w1);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, BN, 1, 1, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1, ab, 102)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(&full[stage], phase, ab, 103)) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        uint64_t da = smem_desc_sw128(sa + kk * 32, 16, 1024);
                        uint64_t db = smem_desc_sw128(sb + kk * 32, 16, 1024);
                        mma_bf16_ss(d_tmem, da, db, idesc, (kb | kk) != 0);
                    }
                    mma_commit(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                mma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int part = warp & 3;                       // TMEM lane partition this warp may read
        const int row_in_tile = part * 32 + lane;
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            if (!mbar_wait(&acc_full[buf], acc_phase, ab, 104)) break;
            tc_fence_after();
            const int row = tm * BM + row_in_tile;
            const uint32_t taddr = tmem_base + (uint32_t(part * 32) << 16) + buf * BN;
            if (p.epilogue == 0) {
                const int col0 = tn * BN;
                __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + col0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
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
            } else {
                const int col0 = tn * 128;
                __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + col0;
#pragma unroll 1
                for (int c = 0; c < 128; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + c, g);
                    tmem_ld32(taddr + 128 + c, u);
                    tmem_wait_ld();
                    if (row < p.m) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (col0 + c + v * 8 < p.n) {
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
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (ab.raised()) {
        // Give copies that are still in flight time to land before the CTA's shared memory is released.
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

int bg_gemm_bf16_pair_launch(const CUtensorMap& map_a, const CUtensorMap& map_w, void* out, int64_t ldo, int64_t m,
                             int64_t n, int64_t k, int epilogue, cudaStream_t stream);

extern "C" int bg_gemm_bf16(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo,
                            int64_t m, int64_t n, int64_t k, int epilogue, void* stream) {
    if (m < 0 || n <= 0 || k <= 0 || (epilogue != 0 && epilogue != 1)) {
        bg_set_error("bg_gemm_bf16: bad shape m=%lld n=%lld k=%lld epilogue=%d", (long long)m, (long long)n,
                     (long long)k, epilogue);
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    if ((k % 8) || (n % 8) || (lda % 8) || (ldw % 8) || (ldo % 8) || (epilogue == 1 && (n % 128))) {
        bg_set_error("bg_gemm_bf16: k, n and leading dimensions must be multiples of 8 (GeGLU: n %% 128 == 0)");
        return BG_ERR_ALIGN;
    }
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) {
        bg_set_error("bg_gemm_bf16: pointers must be 16-byte aligned");
        return BG_ERR_ALIGN;
    }
    const int64_t w_rows = epilogue == 1 ? 2 * n : n;
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda * 2};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)w_rows}, str_w[1] = {(uint64_t)ldw * 2};
    uint32_t box_a[2] = {BK, BM}, box_w[2] = {BK, 128};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims_a, str_a, box_a,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, dims_w, str_w, box_w,
                            CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;

    // More than one row tile: CTA pairs (256 x 256 tiles, a third less L2-to-SM traffic per FLOP).
    if (m > BM) return bg_gemm_bf16_pair_launch(map_a, map_w, out, ldo, m, n, k, epilogue, static_cast<cudaStream_t>(stream));

    GemmParams p;
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.epilogue = epilogue; p.ldo = ldo;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.tiles_m = (int)((m + BM - 1) / BM);
    p.tiles_n = epilogue == 1 ? (int)(n / 128) : (int)((n + BN - 1) / BN);
    // Keep one group's activation rows (group_m x 128 x K bf16) at about a third of the 126 MB L2, so
    // that every weight panel is fetched from DRAM once per group instead of once per 16 row-tiles.
    {
        const int64_t panel = int64_t(BM) * k * 2;
        int64_t g = (40ll << 20) / (panel > 0 ? panel : 1);
        p.group_m = (int)(g < 8 ? 8 : (g > 64 ? 64 : g));
    }
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;

    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            bg_set_error("bg_gemm_bf16: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < bg_num_sms() ? tiles : bg_num_sms();
    cudaError_t e = launch_kernel(gemm_bf16_kernel, dim3((unsigned)grid), dim3(THREADS), SMEM_BYTES,
                                  static_cast<cudaStream_t>(stream), 0, map_a, map_w, p);
    if (e != cudaSuccess) {
        bg_set_error("bg_gemm_bf16: launch: %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}
