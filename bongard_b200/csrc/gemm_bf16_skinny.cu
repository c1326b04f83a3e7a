// BF16 contraction for a FEW rows (M <= 256): the single-request serving case, where one
// question of ~150 tokens meets 190 MB of layer weights and the kernel is bound by how fast
// the weights stream from HBM, not by the tensor cores.
//
//   out[M, N] = A[M, K] . W[N, K]^T
//
// The large-M kernels tile the output 256 wide, which leaves 10-20 CTAs streaming a 2560-column
// projection while 130 SMs idle.  Here the work is cut for bandwidth instead:
//
//   * an output tile is all M rows (one or two 128-row accumulators in TMEM) by 128 weight rows
//     (GeGLU: 64 or 80 gate rows + the matching up rows), so every weight byte is fetched once;
//   * K is split across the CTAs of a thread-block cluster (1-8 CTAs, chosen on the host so that
//     tiles x split fills the GPU in one wave); each CTA streams its K slice through a 4-stage
//     TMA ring and accumulates a partial tile in TMEM;
//   * the partial tiles are reduced through distributed shared memory: once every ring of the
//     cluster has drained, each CTA sends column slice r of its fp32 partial straight from
//     tensor memory into a slot in CTA r's shared memory (16-byte remote stores, which are
//     posted - remote loads measured 5x slower), the cluster synchronises, and CTA r sums its
//     slots in rank order - deterministic, no global workspace, no second kernel - applies the
//     epilogue and stores bf16.
//
// Measured on B200 at 128 rows: the K loop runs at the rate the weight stream arrives from HBM
// (skipping the activation loads or the MMAs changes nothing), so the ring is as deep as shared
// memory allows (5-6 stages) to keep more bytes in flight.
#include "common.cuh"

namespace {

using namespace bg;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int MAX_STAGES = 8;
constexpr int TILE_BYTES = BM * BK * 2;     // one 128-row activation tile of a stage, 16 KB
constexpr int RING_BYTES = 208 * 1024;      // the TMA ring; after it has drained, the reduction slots
constexpr int SMEM_BYTES = RING_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int SLOT_BYTES = BM * 16;         // 4 fp32 columns of 128 rows
constexpr int THREADS = 192;
constexpr int ACC_STRIDE = 256;             // TMEM columns between the two row-tile accumulators

struct SkinnyParams {
    int m, n, k;                  // n = output columns
    int epilogue;                 // 0 plain, 1 GeGLU
    int row_tiles;                // 1 or 2
    int bn;                       // weight rows per tile = MMA N (plain: 128; GeGLU: 2 * half)
    int half;                     // GeGLU: gate rows per tile (= output columns per tile)
    int stages, stage_bytes;      // ring depth and bytes per stage (row_tiles * 16 KB + bn * 128)
    int max_units;                // 8-column output units a CTA may own in the reduction
    int64_t ldo;
    __nv_bfloat16* out;
    int32_t* status;
};

__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, const uint32_t* v) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(cluster_addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_skinny_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const SkinnyParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RING_BYTES);
    uint64_t* full = bars;                     // [stages]
    uint64_t* empty = bars + MAX_STAGES;       // [stages]
    uint64_t* acc_full = bars + 2 * MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};
    const int ks = (int)cluster_nctarank();
    const int rank = (int)cluster_ctarank();
    const int tile = blockIdx.x / ks;

    // this CTA's slice of the K loop
    const int kblocks = (p.k + BK - 1) / BK;
    const int kb_lo = (int)((int64_t)rank * kblocks / ks);
    const int kb_hi = (int)((int64_t)(rank + 1) * kblocks / ks);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
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
    // The weights do not depend on the predecessor in the stream (only the activations do), so the first ring
    // fill of weight tiles is requested before the wait for it: under a programmatic launch the ~2 us from the
    // first request to the first byte overlap the predecessor's tail.  Each stage's barrier is armed for the
    // stage's full byte count here; the activation tiles join after the wait.
    const int w0 = p.epilogue == 1 ? tile * p.half : tile * p.bn;
    const int prefilled = min(p.stages, kb_hi - kb_lo);
    if (threadIdx.x == 0) {
        for (int s = 0; s < prefilled; ++s) {
            uint8_t* sb = smem + s * p.stage_bytes + p.row_tiles * TILE_BYTES;
            mbar_expect_tx(&full[s], uint32_t(p.row_tiles * BM + p.bn) * BK * 2);
            tma_load_2d(sb, &map_w, &full[s], (kb_lo + s) * BK, w0);
            if (p.epilogue == 1) tma_load_2d(sb + p.half * BK * 2, &map_w, &full[s], (kb_lo + s) * BK, p.n + w0);
        }
    }
    pdl_wait();                   // the predecessor in the stream has finished; from here on every global buffer may be touched
    pdl_launch_dependents();      // the successor may start its own prologue

    const int part = warp & 3;
    const int row_in_tile = part * 32 + lane;
    const int units = (p.epilogue == 1 ? p.half : p.bn) / 8;        // 8-column output units per tile
    const int out_col0 = tile * (p.epilogue == 1 ? p.half : p.bn);

    // Apply the epilogue to 8 consecutive output columns of one row and store them.
    auto store8 = [&](int row, int unit, const float* a, const float* b) {
        if (row >= p.m) return;
        float h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = p.epilogue == 1 ? gelu_tanh(a[e]) * b[e] : a[e];
        uint4 o;
        o.x = pack_bf16(h[0], h[1]);
        o.y = pack_bf16(h[2], h[3]);
        o.z = pack_bf16(h[4], h[5]);
        o.w = pack_bf16(h[6], h[7]);
        *reinterpret_cast<uint4*>(p.out + int64_t(row) * p.ldo + out_col0 + unit * 8) = o;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb_lo; kb < kb_hi; ++kb) {
                if (!mbar_wait(&empty[stage], phase ^ 1, ab, 301)) break;
                uint8_t* sa = smem + stage * p.stage_bytes;
                uint8_t* sb = sa + p.row_tiles * TILE_BYTES;
                const bool weights_requested = kb - kb_lo < prefilled;       // armed and requested before the wait above
                if (!weights_requested) mbar_expect_tx(&full[stage], uint32_t(p.row_tiles * BM + p.bn) * BK * 2);
                for (int t = 0; t < p.row_tiles; ++t)
                    tma_load_2d(sa + t * TILE_BYTES, &map_a, &full[stage], kb * BK, t * BM);
                if (weights_requested) {
                    // nothing more to ask for
                } else if (p.epilogue == 1) {
                    tma_load_2d(sb, &map_w, &full[stage], kb * BK, w0);
                    tma_load_2d(sb + p.half * BK * 2, &map_w, &full[stage], kb * BK, p.n + w0);
                } else {
                    tma_load_2d(sb, &map_w, &full[stage], kb * BK, w0);
                }
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = instr_desc(BM, (uint32_t)p.bn, 1, 1, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb_lo; kb < kb_hi && ok; ++kb) {
                if (!mbar_wait(&full[stage], phase, ab, 302)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + stage * p.stage_bytes);
                const uint32_t sb = sa + p.row_tiles * TILE_BYTES;
                for (int t = 0; t < p.row_tiles; ++t) {
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        uint64_t da = smem_desc_sw128(sa + t * TILE_BYTES + kk * 32, 16, 1024);
                        uint64_t db = smem_desc_sw128(sb + kk * 32, 16, 1024);
                        mma_bf16_ss(tmem_base + t * ACC_STRIDE, da, db, idesc, (kb != kb_lo) || kk != 0);
                    }
                }
                mma_commit(&empty[stage]);
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
            if (ok) mma_commit(acc_full);
        }
    } else {
        // ------------------------------------------------------------ epilogue without a split (warps 2..5)
        if (mbar_wait(acc_full, 0, ab, 303) && ks == 1) {
            tc_fence_after();
            for (int t = 0; t < p.row_tiles; ++t) {
                const uint32_t taddr = tmem_base + (uint32_t(part * 32) << 16) + t * ACC_STRIDE;
                const int row = t * BM + row_in_tile;
                for (int u = 0; u < units; u += 4) {
                    uint32_t a[32], b[32];
                    tmem_ld32(taddr + u * 8, a);
                    if (p.epilogue == 1) tmem_ld32(taddr + p.half + u * 8, b);
                    tmem_wait_ld();
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        if (u + v < units)
                            store8(row, u + v, reinterpret_cast<const float*>(a) + v * 8,
                                   reinterpret_cast<const float*>(b) + v * 8);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();

    if (ks > 1) {
        // ------------------------------------------------------------ split-K reduction over the cluster
        // Slot of 4 columns x 128 rows: [source rank][row tile][plane: gate|up][unit][half unit][row][4 floats].
        const int planes = p.epilogue == 1 ? 2 : 1;
        auto slot = [&](int src, int t, int plane, int ul, int h) {
            return (uint32_t)((((((src * p.row_tiles + t) * planes + plane) * p.max_units + ul) * 2 + h) * SLOT_BYTES) +
                              row_in_tile * 16);
        };
        const uint32_t base = smem_u32(smem);
        cluster_sync();                                   // every ring of the cluster has drained
        if (warp >= 2 && !ab.raised()) {
            tc_fence_after();
            for (int t = 0; t < p.row_tiles; ++t) {
                const uint32_t taddr = tmem_base + (uint32_t(part * 32) << 16) + t * ACC_STRIDE;
                for (int c = 0; c < p.bn; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const int col = c + q * 4;
                        const int plane = (p.epilogue == 1 && col >= p.half) ? 1 : 0;
                        const int cl = col - plane * p.half;
                        const int unit = cl >> 3;
                        const int owner = ((unit + 1) * ks - 1) / units;      // the rank whose slice holds `unit`
                        const int ul = unit - owner * units / ks;
                        st_cluster_v4(map_to_cta(base + slot(rank, t, plane, ul, (cl >> 2) & 1), (uint32_t)owner),
                                      r + q * 4);
                    }
                }
            }
        }
        cluster_sync();                                   // every slot of this CTA has been written
        if (warp >= 2 && !ab.raised()) {
            const int u_lo = rank * units / ks, u_hi = (rank + 1) * units / ks;
            for (int t = 0; t < p.row_tiles; ++t) {
                const int row = t * BM + row_in_tile;
                for (int u = u_lo; u < u_hi; ++u) {
                    float a[8], b[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] = b[e] = 0.f;
                    for (int src = 0; src < ks; ++src) {           // rank order: the sum is deterministic
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const float4 va = *reinterpret_cast<const float4*>(smem + slot(src, t, 0, u - u_lo, h));
                            a[h * 4 + 0] += va.x; a[h * 4 + 1] += va.y; a[h * 4 + 2] += va.z; a[h * 4 + 3] += va.w;
                            if (p.epilogue == 1) {
                                const float4 vb = *reinterpret_cast<const float4*>(smem + slot(src, t, 1, u - u_lo, h));
                                b[h * 4 + 0] += vb.x; b[h * 4 + 1] += vb.y; b[h * 4 + 2] += vb.z; b[h * 4 + 3] += vb.w;
                            }
                        }
                    }
                    store8(row, u, a, b);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
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

int max_clusters(int ks) {
    static int cached[9] = {0};
    if (cached[ks]) return cached[ks];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(ks * (bg_num_sms() / ks)));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)ks;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_skinny_kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = bg_num_sms() / ks / 2;                        // conservative guess
        if (n < 1) n = 1;
    }
    cached[ks] = n;
    return n;
}

}  // namespace

static bool skinny_takes(int64_t m, int64_t n, int64_t k, int epilogue) {
    if (m <= 0 || m > 2 * BM || k <= 0 || k % BK || n <= 0) return false;
    return epilogue == 1 ? n % 64 == 0 : n % 128 == 0;
}

// 1 when bg_gemm_bf16_skinny takes the shape, else 0.
extern "C" int bg_gemm_bf16_skinny_supported(int64_t m, int64_t n, int64_t k, int epilogue) {
    return skinny_takes(m, n, k, epilogue) ? 1 : 0;
}

extern "C" int bg_gemm_bf16_skinny(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo,
                                   int64_t m, int64_t n, int64_t k, int epilogue, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if ((epilogue != 0 && epilogue != 1) || !skinny_takes(m, n, k, epilogue)) {
        bg_set_error("bg_gemm_bf16_skinny: takes 1..256 rows, k %% 64 == 0 and n %% 128 == 0 (GeGLU: n %% 64 == 0); "
                     "got m=%lld n=%lld k=%lld epilogue=%d", (long long)m, (long long)n, (long long)k, epilogue);
        return BG_ERR_SHAPE;
    }
    if ((lda % 8) || (ldw % 8) || (ldo % 8) ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15)) {
        bg_set_error("bg_gemm_bf16_skinny: pointers must be 16-byte aligned and leading dimensions multiples of 8");
        return BG_ERR_ALIGN;
    }
    SkinnyParams p;
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.epilogue = epilogue; p.ldo = ldo;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.row_tiles = (int)((m + BM - 1) / BM);
    int tiles;
    if (epilogue == 1) {
        p.half = (n % 80 == 0 && n / 80 <= bg_num_sms()) ? 80 : 64;
        p.bn = 2 * p.half;
        tiles = (int)(n / p.half);
    } else {
        p.half = 0;
        p.bn = 128;
        tiles = (int)(n / 128);
    }

    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES);
        if (e != cudaSuccess) {
            bg_set_error("bg_gemm_bf16_skinny: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }

    p.stage_bytes = p.row_tiles * TILE_BYTES + ((p.bn * BK * 2 + 1023) & ~1023);
    p.stages = RING_BYTES / p.stage_bytes < MAX_STAGES ? RING_BYTES / p.stage_bytes : MAX_STAGES;

    // Split K over 1-8 CTAs of a cluster: fewest waves first, then the shortest K slice; a split pays
    // for its reduction with about 4 K-blocks of time, every CTA for about 8 of fixed cost.  The
    // reduction slots of a CTA (one per source rank) must fit the drained ring.
    const int kblocks = (int)(k / BK);
    const int units = (epilogue == 1 ? p.half : p.bn) / 8;
    int best_ks = 1;
    int64_t best_cost = INT64_MAX;
    for (int ks = 1; ks <= 8; ++ks) {
        if (ks > kblocks) break;
        const int max_units = (units + ks - 1) / ks;
        if (ks > 1 && ks * p.row_tiles * (epilogue == 1 ? 2 : 1) * max_units * 2 * SLOT_BYTES > RING_BYTES) continue;
        const int resident = max_clusters(ks);
        const int waves = (tiles + resident - 1) / resident;
        const int64_t cost = int64_t(waves) * ((kblocks + ks - 1) / ks + 8 + (ks > 1 ? 4 : 0));
        if (cost < best_cost) { best_cost = cost; best_ks = ks; }
    }

    CUtensorMap map_a, map_w;
    const int64_t w_rows = epilogue == 1 ? 2 * n : n;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda * 2};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)w_rows}, str_w[1] = {(uint64_t)ldw * 2};
    uint32_t box_a[2] = {BK, BM}, box_w[2] = {BK, (uint32_t)(epilogue == 1 ? p.half : p.bn)};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims_a, str_a, box_a,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, dims_w, str_w, box_w,
                            CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;

    p.max_units = (units + best_ks - 1) / best_ks;

    cudaError_t e = launch_kernel(gemm_bf16_skinny_kernel, dim3((unsigned)(tiles * best_ks)), dim3(THREADS), SMEM_BYTES,
                                  stream, best_ks, map_a, map_w, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        bg_set_error("bg_gemm_bf16_skinny: launch (%d tiles x %d): %s", tiles, best_ks, cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}
