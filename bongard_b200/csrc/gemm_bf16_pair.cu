// BF16 contraction on CTA PAIRS (thread-block cluster of 2, tcgen05 cta_group::2).
//
//   out[M, N] = A[M, K] . W[N, K]^T, output tile 256 x 256 per pair.
//
// Why pairs: a single-CTA 128 x 256 tile has to pull 48 KB (A 16 KB + W 32 KB) from L2 into its
// SM for every 512 tensor-core clocks, and that L2-to-SM stream, not the tensor pipe, is what
// limits the single-CTA kernel.  In a pair each CTA loads its own 128 rows of A and only HALF
// of the weight panel (128 of the 256 rows); one tcgen05.mma.cta_group::2 instruction issued
// by the leader CTA drives both tensor cores with M = 256 and reads the two weight halves
// from both CTAs' shared memory.  Per CTA that is 32 KB per 512 clocks - a third less.
//
// A stage covers 128 of the contraction (two 64-element swizzle slabs per operand, 64 KB per CTA, three
// stages).  Issuing one MMA costs the issuing thread ~65 cycles, a barrier test ~70 and the two commits
// that free a stage ~120, so with 64-deep stages (4 MMAs of 128 tensor-core cycles each) the thread
// needed ~630 cycles per 512 cycles of tensor work and the pipe idled for a sixth of the time; with
// 8 MMAs per stage the same overheads fit under the 1024 cycles the pipe needs.
//
// Synchronisation between the two CTAs (all barriers sit at the same shared-memory offset in
// both CTAs; nothing uses a multi-destination form):
//   full[s]       leader only.  Both CTAs' TMA loads credit their bytes to the leader's barrier.
//   empty[s]      one per CTA.  The leader commits twice: to its own barrier and to the peer's.
//   acc_full[b]   one per CTA, same double commit.
//   acc_empty[b]  leader only, 8 arrivals: 4 epilogue warps of each CTA (the peer arrives remotely).
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer (leader only), warps 2-5 epilogue.
#include "common.cuh"

namespace {

using namespace bg;

constexpr int BM = 128;           // rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 128;           // contraction per stage: two 64-element (128-byte) swizzle slabs
constexpr int STAGES = 3;
constexpr int A_BYTES = BM * BK * 2;        // 32 KB
constexpr int B_BYTES = (BN / 2) * BK * 2;  // 32 KB: this CTA's half of the weight panel
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + 2 * 256 * 4;
constexpr int THREADS = 192;

struct PairParams {
    int m, n, k, epilogue;
    int64_t ldo;
    __nv_bfloat16* out;
    int tiles_m, tiles_n;         // in units of 256-row pair tiles
    int group_m;
    int32_t* status;
    // epilogue 3 (split-K): work item = (tile, K slice); fp32 partial tiles [split_k, m, n] summed by a second kernel
    int split_k;
    float* partial;
    int mn_major;                 // host side only: selects the MN-major instantiation
    // epilogue 2 (q|k|v projection with QK-norm + RoPE)
    int q_dim, kv_dim, head_dim, table_rows;
    float eps;
    const __nv_bfloat16* q_gain;  // [head_dim] RMSNorm weights w (the gain is 1 + w)
    const __nv_bfloat16* k_gain;
    const int32_t* positions;     // [m]
    const float2* rope_table;     // [table_rows, head_dim / 2] (cos, sin)
};

constexpr int GAIN_BYTES = 2 * 256 * 4;     // (1 + w) of the q and k norms as fp32, after the barriers

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
    int per_group = group_m * tiles_n;
    int group = tile / per_group;
    int first_m = group * group_m;
    int rows = min(group_m, tiles_m - first_m);
    int in_group = tile - group * per_group;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
}

// MN = true is the weight-gradient form: out[M, N] = sum_k At[k, M] * Wt[k, N] with both operands stored
// with the contraction as the ROW index (dW = dy^T x straight from dy [tokens, out] and x [tokens, in]).
// A stage then holds, per operand, two slabs of 128 contraction rows x 64 elements (128 B, swizzled) instead of
// two slabs of 128 rows x 64 contraction elements, and the MMA descriptors say "MN-major".
template <bool MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                        // [STAGES]
    uint64_t* empty = bars + STAGES;              // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;       // [2]
    uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const Abort ab{abort_flag, p.status};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);
        }
        mbar_fence_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();               // both CTAs' barriers are initialised before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                   // the predecessor in the stream has finished; from here on global memory may be touched
    pdl_launch_dependents();      // the successor may start its own prologue
    float* gains = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256);   // [2][256]: q, k
    if (p.epilogue == 2 && warp >= 2) {
        for (int i = threadIdx.x - 64; i < 2 * p.head_dim; i += 128) {
            const bool is_k = i >= p.head_dim;
            gains[(is_k ? 256 : 0) + (is_k ? i - p.head_dim : i)] =
                1.f + __bfloat162float((is_k ? p.k_gain : p.q_gain)[is_k ? i - p.head_dim : i]);
        }
        named_barrier(1, 128);
    }

    const int pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
    // With split-K the work list is num_tiles * split_k items: item i covers K-blocks
    // [slice * kblocks / split_k, (slice + 1) * kblocks / split_k) of tile i % tiles, slice = i / tiles.
    const int mn_tiles = p.tiles_m * p.tiles_n;
    const int num_tiles = mn_tiles * p.split_k;
    const int kblocks = (p.k + BK - 1) / BK;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = pair; tile < num_tiles; tile += pairs) {
                int tm, tn;
                tile_coords(tile % mn_tiles, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
                const int slice = tile / mn_tiles;
                const int kb0 = slice * kblocks / p.split_k, kb1 = (slice + 1) * kblocks / p.split_k;
                const int row0 = tm * 2 * BM + rank * BM;
                // this CTA's half of the weight panel: plain -> columns [256 tn + 128 rank, +128);
                // GeGLU -> rank 0 loads 128 gate rows, rank 1 the matching 128 up rows.
                const int w0 = p.epilogue == 1 ? (rank == 0 ? tn * 128 : p.n + tn * 128) : tn * BN + rank * 128;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_parked(&empty[stage], phase ^ 1, ab, 111)) break;
                    uint8_t* sa = smem + stage * STAGE_BYTES;
                    const uint32_t leader_full = map_to_cta(smem_u32(&full[stage]), 0);
                    if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
                    if constexpr (MN) {
                        tma_load_2d_pair(sa, &map_a, leader_full, row0, kb * BK);
                        tma_load_2d_pair(sa + A_BYTES / 2, &map_a, leader_full, row0 + 64, kb * BK);
                        tma_load_2d_pair(sa + A_BYTES, &map_w, leader_full, w0, kb * BK);
                        tma_load_2d_pair(sa + A_BYTES + B_BYTES / 2, &map_w, leader_full, w0 + 64, kb * BK);
                    } else {
                        tma_load_2d_pair(sa, &map_a, leader_full, kb * BK, row0);
                        tma_load_2d_pair(sa + A_BYTES, &map_w, leader_full, kb * BK, w0);
                        tma_load_2d_pair(sa + A_BYTES / 2, &map_a, leader_full, kb * BK + 64, row0);
                        tma_load_2d_pair(sa + A_BYTES + B_BYTES / 2, &map_w, leader_full, kb * BK + 64, w0);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = instr_desc(2 * BM, BN, 1, 1, MN ? 1 : 0, MN ? 1 : 0);
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            for (int tile = pair; tile < num_tiles; tile += pairs, ++local) {
                const int buf = local & 1;
                if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, ab, 112)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int slice = tile / mn_tiles;
                const int kb0 = slice * kblocks / p.split_k, kb1 = (slice + 1) * kblocks / p.split_k;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, ab, 113)) break;
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // K-major: 32 B along the swizzled row per 16-deep step, the second 64 of the contraction in
                        // the second slab; MN-major: 16 contraction rows of 128 B per step, slabs of 64 elements
                        // half an operand apart
                        uint64_t da = MN ? smem_desc_sw128(sa + kk * 2048, A_BYTES / 2, 1024)
                                         : smem_desc_sw128(sa + (kk >> 2) * (A_BYTES / 2) + (kk & 3) * 32, 16, 1024);
                        uint64_t db = MN ? smem_desc_sw128(sb + kk * 2048, B_BYTES / 2, 1024)
                                         : smem_desc_sw128(sb + (kk >> 2) * (B_BYTES / 2) + (kk & 3) * 32, 16, 1024);
                        mma_bf16_ss_pair(d_tmem, da, db, idesc, kb != kb0 || kk != 0);
                    }
                    const uint32_t e = smem_u32(&empty[stage]);
                    mma_commit_pair(map_to_cta(e, 0));
                    mma_commit_pair(map_to_cta(e, 1));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                const uint32_t f = smem_u32(&acc_full[buf]);
                mma_commit_pair(map_to_cta(f, 0));
                mma_commit_pair(map_to_cta(f, 1));
            }
        }
    } else {
        const int part = warp & 3;
        const int row_in_tile = part * 32 + lane;
        int local = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++local) {
            int tm, tn;
            tile_coords(tile % mn_tiles, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
            const int buf = local & 1;
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, ab, 114)) break;
            tc_fence_after();
            const int row = tm * 2 * BM + rank * BM + row_in_tile;
            const uint32_t taddr = tmem_base + (uint32_t(part * 32) << 16) + buf * BN;
            if (p.epilogue == 2) {
                // q|k|v projection: every head of this 256-column tile is complete in this thread's TMEM lane.
                // Query and key heads get the RMSNorm over the head with gain (1 + w) and the rotate-half RoPE
                // of the token's position (bongard/attention.py:172-180) before the one rounding to bf16;
                // the projection itself is rounded to bf16 first, as the module chain does.  Value heads are
                // stored as they are.
                const int col0 = tn * BN;
                const int D = p.head_dim, HD = D >> 1;
                int pos = row < p.m ? p.positions[row] : 0;
                pos = pos < 0 ? 0 : (pos >= p.table_rows ? p.table_rows - 1 : pos);
                const float2* trow = p.rope_table + int64_t(pos) * HD;
#pragma unroll 1
                for (int hb = 0; hb < BN; hb += D) {
                    const int hcol = col0 + hb;                       // first output column of this head
                    if (hcol >= p.n) break;
                    __nv_bfloat16* dst = p.out + int64_t(row) * p.ldo + hcol;
                    if (hcol >= p.q_dim + p.kv_dim) {
                        // value head: plain store
#pragma unroll 1
                        for (int c = 0; c < D; c += 32) {
                            uint32_t r[32];
                            tmem_ld32(taddr + hb + c, r);
                            tmem_wait_ld();
                            if (row < p.m) {
#pragma unroll
                                for (int v = 0; v < 4; ++v) {
                                    uint4 o;
                                    o.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                                    o.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                                    o.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                                    o.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                                    *reinterpret_cast<uint4*>(dst + c + v * 8) = o;
                                }
                            }
                        }
                        continue;
                    }
                    const float* gain = gains + (hcol >= p.q_dim ? 256 : 0);
                    float ss = 0.f;
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(taddr + hb + c, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float x = round_bf16(__uint_as_float(r[i]));
                            ss += x * x;
                        }
                    }
                    const float rinv = rsqrtf(ss / float(D) + p.eps);
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t lo[32], hi[32];
                        tmem_ld32(taddr + hb + c, lo);
                        tmem_ld32(taddr + hb + HD + c, hi);
                        tmem_wait_ld();
                        if (row < p.m) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                float ol[8], oh[8];
#pragma unroll
                                for (int q4 = 0; q4 < 4; ++q4) {
                                    // two (cos, sin) pairs per 16-byte load
                                    const float4 t = __ldg(reinterpret_cast<const float4*>(trow + c + v * 8 + q4 * 2));
#pragma unroll
                                    for (int e2 = 0; e2 < 2; ++e2) {
                                        const int i = v * 8 + q4 * 2 + e2;
                                        const float cs = e2 ? t.z : t.x, sn = e2 ? t.w : t.y;
                                        const float a = round_bf16(__uint_as_float(lo[i])) * rinv * gain[c + i];
                                        const float b = round_bf16(__uint_as_float(hi[i])) * rinv * gain[HD + c + i];
                                        ol[q4 * 2 + e2] = a * cs - b * sn;
                                        oh[q4 * 2 + e2] = b * cs + a * sn;
                                    }
                                }
                                uint4 o;
                                o.x = pack_bf16(ol[0], ol[1]); o.y = pack_bf16(ol[2], ol[3]);
                                o.z = pack_bf16(ol[4], ol[5]); o.w = pack_bf16(ol[6], ol[7]);
                                *reinterpret_cast<uint4*>(dst + c + v * 8) = o;
                                o.x = pack_bf16(oh[0], oh[1]); o.y = pack_bf16(oh[2], oh[3]);
                                o.z = pack_bf16(oh[4], oh[5]); o.w = pack_bf16(oh[6], oh[7]);
                                *reinterpret_cast<uint4*>(dst + HD + c + v * 8) = o;
                            }
                        }
                    }
                }
            } else if (p.epilogue == 3) {
                // split-K: this item's fp32 partial sums, unrounded
                const int col0 = tn * BN;
                float* dst = p.partial + (int64_t(tile / mn_tiles) * p.m + row) * p.n + col0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_wait_ld();
                    if (row < p.m) {
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            if (col0 + c + v * 4 < p.n)
                                *reinterpret_cast<uint4*>(dst + c + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
                        }
                    }
                }
            } else if (p.epilogue == 0) {
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
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        }
    }

    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    tc_fence_before();
    __syncthreads();
    if (ab.raised()) {
        uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// out[r, c] = bf16(sum over slices of partial[slice, r, c]); eight columns per thread (n % 8 == 0).
__global__ void sum_partials_kernel(const float* __restrict__ partial, int split, int64_t m, int64_t n,
                                    __nv_bfloat16* __restrict__ out, int64_t ldo) {
    pdl_wait();
    const int64_t i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i >= m * n) return;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < split; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(partial + s * m * n + i);
        const float4 b = *reinterpret_cast<const float4*>(partial + s * m * n + i + 4);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (i / n) * ldo + i % n) = o;
}

}  // namespace

static int pair_launch(PairParams p, const CUtensorMap& map_a, const CUtensorMap& map_w, void* out, int64_t ldo,
                       int64_t m, int64_t n, int64_t k, int epilogue, cudaStream_t stream);

// Launcher used by bg_gemm_bf16 for every problem with more than 128 rows.
int bg_gemm_bf16_pair_launch(const CUtensorMap& map_a, const CUtensorMap& map_w, void* out, int64_t ldo, int64_t m,
                             int64_t n, int64_t k, int epilogue, cudaStream_t stream) {
    PairParams p = {};
    return pair_launch(p, map_a, map_w, out, ldo, m, n, k, epilogue, stream);
}

// out[m, q_dim + 2 kv_dim] = a . w^T with QK-norm + RoPE applied to the query and key heads in the epilogue.
extern "C" int bg_gemm_bf16_qkv_rope(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo,
                                     int64_t m, int64_t k, int q_dim, int kv_dim, int head_dim, const void* q_gain,
                                     const void* k_gain, const int32_t* positions, const float* rope_table,
                                     int64_t table_rows, float eps, void* stream) {
    const int64_t n = int64_t(q_dim) + 2 * int64_t(kv_dim);
    if (m < 0 || k <= 0 || q_dim <= 0 || kv_dim <= 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256) ||
        q_dim % head_dim || kv_dim % head_dim || table_rows <= 0) {
        bg_set_error("bg_gemm_bf16_qkv_rope: bad shape (q_dim %d, kv_dim %d, head_dim %d)", q_dim, kv_dim, head_dim);
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    if ((k % 8) || (lda % 8) || (ldw % 8) || (ldo % 8) ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
          reinterpret_cast<uintptr_t>(rope_table)) & 15)) {
        bg_set_error("bg_gemm_bf16_qkv_rope: pointers must be 16-byte aligned, k and leading dimensions multiples of 8");
        return BG_ERR_ALIGN;
    }
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda * 2};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)n}, str_w[1] = {(uint64_t)ldw * 2};
    uint32_t box_a[2] = {64, BM}, box_w[2] = {64, 128};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims_a, str_a, box_a,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, dims_w, str_w, box_w,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    PairParams p = {};
    p.q_dim = q_dim; p.kv_dim = kv_dim; p.head_dim = head_dim; p.table_rows = (int)table_rows; p.eps = eps;
    p.q_gain = static_cast<const __nv_bfloat16*>(q_gain);
    p.k_gain = static_cast<const __nv_bfloat16*>(k_gain);
    p.positions = positions;
    p.rope_table = reinterpret_cast<const float2*>(rope_table);
    return pair_launch(p, map_a, map_w, out, ldo, m, n, k, 2, static_cast<cudaStream_t>(stream));
}

// Number of CTA pairs that can be resident at once (pairs must sit inside one GPC, so it can be
// fewer than SMs / 2); the persistent grid is sized to it so that every pair starts immediately.
static int resident_pairs() {
    static int max_pairs = 0;
    if (!max_pairs) {
        cudaFuncSetAttribute(gemm_bf16_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (bg_num_sms() / 2));
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = bg_num_sms() / 2;
        }
        max_pairs = n < bg_num_sms() / 2 ? n : bg_num_sms() / 2;
    }
    return max_pairs;
}

static int pair_launch(PairParams p, const CUtensorMap& map_a, const CUtensorMap& map_w, void* out, int64_t ldo,
                       int64_t m, int64_t n, int64_t k, int epilogue, cudaStream_t stream) {
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.epilogue = epilogue; p.ldo = ldo;
    if (p.split_k < 1) p.split_k = 1;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.tiles_m = (int)((m + 2 * BM - 1) / (2 * BM));
    p.tiles_n = epilogue == 1 ? (int)(n / 128) : (int)((n + BN - 1) / BN);
    {
        // Raster: the tiles of `group_m` row panels x all column panels run before the next group.  With many
        // column panels (gate | up: 80) a group holds as many activation rows as stay in L2 (~40 MB) while the
        // weight streams past once per group.  With few (the q|k|v, output and down projections: 10 - 16) one
        // wave of the grid already spans several row panels, and small groups measured best (DRAM reads of the
        // down projection at 32 768 rows: 2.8 GB with 7 panels per group, 2.0 - 2.2 GB with 2 - 4).
        const int64_t panel = int64_t(2 * BM) * k * 2;
        int64_t g = (40ll << 20) / (panel > 0 ? panel : 1);
        p.group_m = (int)(g < 4 ? 4 : (g > 32 ? 32 : g));
        if (p.tiles_n < 32) p.group_m = k >= 8192 ? 3 : 4;
    }
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;
    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_bf16_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            bg_set_error("bg_gemm_bf16: cudaFuncSetAttribute(pair): %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    const int max_pairs = resident_pairs();
    const int tiles = p.tiles_m * p.tiles_n * p.split_k;
    const int pairs = tiles < max_pairs ? tiles : max_pairs;
    cudaError_t e = p.mn_major ? launch_kernel(gemm_bf16_pair_kernel<true>, dim3((unsigned)(2 * pairs)), dim3(THREADS),
                                               SMEM_BYTES, stream, 0, map_a, map_w, p)
                               : launch_kernel(gemm_bf16_pair_kernel<false>, dim3((unsigned)(2 * pairs)), dim3(THREADS),
                                               SMEM_BYTES, stream, 0, map_a, map_w, p);
    if (e != cudaSuccess) {
        bg_set_error("bg_gemm_bf16: launch(pair): %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

// ---------------------------------------------------------------------------------------------------
// Split-K for problems whose 256 x 256 output tiles fill less than half of the machine (a few hundred
// rows against a narrow weight with a long contraction: the down projection of a short request).
// Each (tile, K slice) is one work item of the same persistent kernel; slices write fp32 partial tiles
// to the caller's workspace and a second kernel sums them in slice order and rounds once.

static int splitk_choice(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0 || k < 4096 || n % 8) return 1;
    const int64_t tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
    const int pairs = resident_pairs();
    if (tiles > 3 * pairs) return 1;
    // time ~ waves of the persistent grid x the length of one item: ceil(tiles * s / pairs) / s against
    // ceil(tiles / pairs) unsplit, plus the partial-sum traffic; a split has to save at least 15 % to be taken
    const int64_t kblocks = (k + 63) / 64;          // the split rules count 64-deep blocks
    const double unsplit = double((tiles + pairs - 1) / pairs);
    int best = 1;
    double best_cost = 1.0;
    for (int split = 2; split <= 4 && kblocks >= 16 * split; ++split) {
        const double cost = double((tiles * split + pairs - 1) / pairs) / split / unsplit + 0.03 * (split - 1);
        if (cost < best_cost - 1e-9 && cost <= 0.85) {
            best = split;
            best_cost = cost;
        }
    }
    return best;
}

extern "C" int bg_gemm_bf16_splitk_choice(int64_t m, int64_t n, int64_t k) { return splitk_choice(m, n, k); }

extern "C" int64_t bg_gemm_bf16_splitk_workspace_bytes(int64_t m, int64_t n, int split) {
    return (m <= 0 || n <= 0 || split < 2) ? 0 : int64_t(split) * m * n * int64_t(sizeof(float));
}

extern "C" int bg_gemm_bf16_splitk(const void* a, int64_t lda, const void* w, int64_t ldw, void* out, int64_t ldo,
                                   int64_t m, int64_t n, int64_t k, int split, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
    const int64_t kblocks = (k + 63) / 64;
    if (m < 0 || n <= 0 || k <= 0 || n % 8 || split < 2 || split > 8 || kblocks < 4 * split) {
        bg_set_error("bg_gemm_bf16_splitk: bad shape (n must be a multiple of 8, 2 <= split <= 8 slices of at least 4 K-blocks)");
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    if ((k % 8) || (lda % 8) || (ldw % 8) || (ldo % 8) ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) |
          reinterpret_cast<uintptr_t>(workspace)) & 15)) {
        bg_set_error("bg_gemm_bf16_splitk: pointers must be 16-byte aligned, k and leading dimensions multiples of 8");
        return BG_ERR_ALIGN;
    }
    if (workspace == nullptr || workspace_bytes < bg_gemm_bf16_splitk_workspace_bytes(m, n, split)) {
        bg_set_error("bg_gemm_bf16_splitk: the workspace is too small");
        return BG_ERR_WORKSPACE;
    }
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda * 2};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)n}, str_w[1] = {(uint64_t)ldw * 2};
    uint32_t box_a[2] = {64, BM}, box_w[2] = {64, 128};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims_a, str_a, box_a,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, dims_w, str_w, box_w,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    PairParams p = {};
    p.split_k = split;
    p.partial = static_cast<float*>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = pair_launch(p, map_a, map_w, out, ldo, m, n, k, 3, s);
    if (rc) return rc;
    const int64_t groups = m * n / 8;
    cudaError_t e = launch_kernel(sum_partials_kernel, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, s, 0,
                                  static_cast<const float*>(workspace), split, m, n, static_cast<__nv_bfloat16*>(out), ldo);
    if (e != cudaSuccess) {
        bg_set_error("bg_gemm_bf16_splitk: launch(sum): %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

// out[m, n] = a . w^T as UNROUNDED fp32 (contiguous [m, n]): the plain GEMM with the accumulators written as they
// are.  Feeds the post-norm of a layer whose residual stream is kept in fp32.
extern "C" int bg_gemm_bf16_f32out(const void* a, int64_t lda, const void* w, int64_t ldw, float* out, int64_t m,
                                   int64_t n, int64_t k, void* stream) {
    if (m < 0 || n <= 0 || k <= 0 || n % 8) {
        bg_set_error("bg_gemm_bf16_f32out: bad shape (n must be a multiple of 8)");
        return BG_ERR_SHAPE;
    }
    if (m == 0) return BG_OK;
    if ((k % 8) || (lda % 8) || (ldw % 8) ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15)) {
        bg_set_error("bg_gemm_bf16_f32out: pointers must be 16-byte aligned, k and leading dimensions multiples of 8");
        return BG_ERR_ALIGN;
    }
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)k, (uint64_t)m}, str_a[1] = {(uint64_t)lda * 2};
    uint64_t dims_w[2] = {(uint64_t)k, (uint64_t)n}, str_w[1] = {(uint64_t)ldw * 2};
    uint32_t box_a[2] = {64, BM}, box_w[2] = {64, 128};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, dims_a, str_a, box_a,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w, dims_w, str_w, box_w,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    PairParams p = {};
    p.split_k = 1;
    p.partial = out;             // one K slice: its "partial" tile is the result
    return pair_launch(p, map_a, map_w, nullptr, n, m, n, k, 3, static_cast<cudaStream_t>(stream));
}

// out[m, n] = sum_k at[k, m] * wt[k, n]: both operands with the contraction as the row index.  This is the
// weight gradient dW = dy^T x taken straight from dy [tokens, out features] and x [tokens, in features].
extern "C" int bg_gemm_bf16_tn(const void* at, int64_t ldat, const void* wt, int64_t ldwt, void* out, int64_t ldo,
                               int64_t m, int64_t n, int64_t k, int split, void* workspace, int64_t workspace_bytes,
                               void* stream) {
    if (m <= 0 || n <= 0 || k <= 0 || split > 8) {
        bg_set_error("bg_gemm_bf16_tn: bad shape");
        return BG_ERR_SHAPE;
    }
    if (split < 2) split = 1;
    if ((m % 8) || (n % 8) || (ldat % 8) || (ldwt % 8) || (ldo % 8) || ldat < m || ldwt < n || ldo < n ||
        ((reinterpret_cast<uintptr_t>(at) | reinterpret_cast<uintptr_t>(wt) | reinterpret_cast<uintptr_t>(out)) & 15) ||
        (split > 1 && (reinterpret_cast<uintptr_t>(workspace) & 15))) {
        bg_set_error("bg_gemm_bf16_tn: pointers must be 16-byte aligned, m, n and the leading dimensions multiples of 8");
        return BG_ERR_ALIGN;
    }
    if (split > 1 && ((k + 63) / 64 < 4 * split || workspace == nullptr ||
                      workspace_bytes < bg_gemm_bf16_splitk_workspace_bytes(m, n, split))) {
        bg_set_error("bg_gemm_bf16_tn: K slices need at least 4 K-blocks each and a workspace of split * m * n * 4 bytes");
        return BG_ERR_WORKSPACE;
    }
    CUtensorMap map_a, map_w;
    uint64_t dims_a[2] = {(uint64_t)m, (uint64_t)k}, str_a[1] = {(uint64_t)ldat * 2};
    uint64_t dims_w[2] = {(uint64_t)n, (uint64_t)k}, str_w[1] = {(uint64_t)ldwt * 2};
    uint32_t box[2] = {64, BK};
    int rc = bg_make_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, at, dims_a, str_a, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = bg_make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, wt, dims_w, str_w, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    PairParams p = {};
    p.mn_major = 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (split == 1) return pair_launch(p, map_a, map_w, out, ldo, m, n, k, 0, s);
    p.split_k = split;
    p.partial = static_cast<float*>(workspace);
    rc = pair_launch(p, map_a, map_w, out, ldo, m, n, k, 3, s);
    if (rc) return rc;
    const int64_t groups = m * n / 8;
    cudaError_t e = launch_kernel(sum_partials_kernel, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, s, 0,
                                  static_cast<const float*>(workspace), split, m, n, static_cast<__nv_bfloat16*>(out), ldo);
    if (e != cudaSuccess) {
        bg_set_error("bg_gemm_bf16_tn: launch(sum): %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}
