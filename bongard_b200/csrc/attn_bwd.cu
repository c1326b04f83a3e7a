// Backward of the packed variable-length attention (bongard/flash_varlen.py:30-39, 85-105:
// `flash_packed_backward`, `flash_prefix_backward`) on tcgen05 tensor cores.
//
// With P = softmax(scale * Q K^T) restricted to each row's visible keys, delta = rowsum(dO * O):
//     dV = P^T dO          dP = dO V^T          dS = scale * P * (dP - delta)
//     dQ = dS K            dK = dS^T Q
// P is recomputed from the saved log-sum-exp, never stored.  Head size 256 leaves no room in
// tensor memory (512 columns) for dK, dV and the score tiles at once, so the work is three passes
// of ONE kernel template, each the shape of the forward kernel - a resident 128-row tile, tiles
// streamed past it (64 rows where two resident tiles fill shared memory, 128 rows for dV), scores
// in TMEM, the elementwise step by eight warps (two per TMEM lane quadrant, half of the score
// columns each), its result written back to TMEM as bf16 and consumed from there by a TS-form MMA:
//
//   pass   resident (X1, X2)    streamed (Y1, Y2)     A1 = X1 Y1^T   A2 = X2 Y2^T   OUT += E * B
//   DQ     Q tile, dO tile      K, V key tiles        S              dP             dS   * K (Y1)
//   DK     K tile, V tile       Q, dO row tiles       S^T            dP^T           dS^T * Q (Y1)
//   DV     K tile               Q, dO row tiles       S^T            -              P^T  * dO (Y2)
//
// DQ walks the forward's query tiles (state prefix first, then own keys); DK and DV walk key
// tiles - own keys against the queries that can see them, state keys against every query of the
// owner's questions - and write dK/dV (or the state's dK/dV) exactly once, so nothing is
// accumulated with atomics and the result is deterministic.  GQA: a query-type tile holds
// (token, head-in-group) rows, so the sum over the heads of a group happens inside the MMA.
#include "common.cuh"
#include <climits>

namespace {

using namespace bg;

constexpr int ROWS = 128;          // resident rows (TMEM lanes)
constexpr int THREADS = 320;       // warp 0 TMA, warp 1 MMA, warps 2-9 elementwise (two per TMEM lane quadrant)
constexpr int EW_WARPS = 8;
constexpr int SLAB_RES = ROWS * 128;      // one 64-column slab of a resident tile
constexpr float LOG2E = 1.4426950408889634f;

enum Pass { DQ = 0, DK = 1, DV = 2 };

struct BwdParams {
    const int32_t* tiles;     // DQ: forward tiles [n][8]; DK/DV: key tiles [n][8] {k_start k_count q_lo q_hi is_prefix}
    const int32_t* row_lo;    // [Tq] own-key range of every query token
    const int32_t* row_hi;
    const float* lse;         // [Hq, Tq] natural-log LSE of the scaled scores (forward output)
    const float* delta;       // [Hq, Tq] rowsum(dO * O)
    __nv_bfloat16* out;       // DQ: dq [Tq, Hq, D]; DK/DV: dk/dv [Tk, Hkv, D]
    __nv_bfloat16* out_state; // DK/DV: state dk/dv [Ts, Hkv, D]
    int64_t tq;
    int q_heads, kv_heads;
    float scale;
    int32_t* status;
};

// Shared memory.  DQ and DK keep two resident tiles (128 KB at head size 256), which leaves room for
// 64-row streamed tiles only: Y1 (needed by the score MMA and by OUT) in two slots, Y2 (needed by
// the second score MMA only) in one.  DV keeps one resident tile and streams 128-row tiles through
// one slot each, the forward kernel's budget.
template <int D, int PASS>
struct Layout {
    static constexpr int SLABS = D / 64;
    static constexpr int SR = PASS == DV ? 128 : 64;                  // streamed rows per iteration
    static constexpr int SLAB_STR = SR * 128;
    static constexpr int RES = SLABS * SLAB_RES;
    static constexpr int STR = SLABS * SLAB_STR;
    static constexpr int NY1 = PASS == DV ? 1 : 2;
    static constexpr int X1 = 0;
    static constexpr int X2 = X1 + RES;
    static constexpr int Y1 = PASS == DV ? X1 + RES : X2 + RES;
    static constexpr int Y2 = Y1 + NY1 * STR;
    static constexpr int COLS = Y2 + STR;                             // per-column facts of two streamed tiles
    static constexpr int BARS = COLS + 2 * SR * 16;
    static constexpr int TOTAL = BARS + 256;
};

struct ColInfo {                   // per streamed query row (DK/DV)
    float lse2, delta;
    int lo, hi;
};

template <int D, int PASS>
__global__ void __launch_bounds__(THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap map_x1, const __grid_constant__ CUtensorMap map_x2,
                     const __grid_constant__ CUtensorMap map_cx1, const __grid_constant__ CUtensorMap map_cx2,
                     const __grid_constant__ CUtensorMap map_y1, const __grid_constant__ CUtensorMap map_y2,
                     const __grid_constant__ CUtensorMap map_cy1, const __grid_constant__ CUtensorMap map_cy2,
                     const BwdParams p) {
    using L = Layout<D, PASS>;
    constexpr int SLABS = L::SLABS;
    constexpr int SR = L::SR;
    constexpr int HALF = SR / 2;        // streamed rows (score columns) one elementwise warp handles
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint64_t* x_full = bars + 0;
    uint64_t* y1_full = bars + 1;    // [2]
    uint64_t* y1_empty = bars + 3;   // [2]
    uint64_t* y2_full = bars + 5;
    uint64_t* y2_empty = bars + 6;
    uint64_t* a_full = bars + 7;     // [2]
    uint64_t* e_full = bars + 9;     // 8 warp arrivals
    uint64_t* out_done = bars + 10;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    ColInfo* cols = reinterpret_cast<ColInfo*>(smem + L::COLS);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};
    const int kvh = blockIdx.y;
    const int G = p.q_heads / p.kv_heads;

    const int32_t* t = p.tiles + int64_t(blockIdx.x) * 8;
    // DQ: the forward tile record.  DK/DV: a key tile.
    const int t0 = t[0], t1 = t[1], t2 = t[2], t3 = t[3], t4 = t[4], t6 = t[6], t7 = t[7];
    int n_pre = 0, n_iter = 0;
    if (PASS == DQ) {
        n_pre = (t7 + SR - 1) / SR;
        n_iter = n_pre + (t3 - t2 + SR - 1) / SR;
    } else {
        const int per = SR / G;                          // query tokens per streamed tile
        n_iter = (t3 - t2 + per - 1) / per;
    }
    const bool state_tile = PASS != DQ && t4 != 0;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        if ((smem_u32(smem) & 1023u) != 0) ab.raise(400);      // the swizzled tiles need a 1024-byte base
        mbar_init(x_full, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&y1_full[b], 1);
            mbar_init(&y1_empty[b], 1);
            mbar_init(&a_full[b], 1);
        }
        mbar_init(y2_full, 1);
        mbar_init(y2_empty, 1);
        mbar_init(e_full, EW_WARPS);
        mbar_init(out_done, 1);
        mbar_fence_init();
        tma_prefetch_desc(&map_x1);
        tma_prefetch_desc(&map_y1);
        tma_prefetch_desc(&map_y2);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_out = tmem_base + 256;
    // score buffers: A1[b] at column b * SR; A2[b] (DQ/DK, SR = 64) at 128 + b * SR
    const bool run = n_iter > 0 && !ab.raised();

    // First streamed row (key or query token) of iteration j, and whether it comes from the state tensors.
    auto stream_origin = [&](int j, bool& from_state) {
        if (PASS == DQ) {
            from_state = j < n_pre;
            return from_state ? t6 + j * SR : t2 + (j - n_pre) * SR;
        }
        from_state = false;
        return t2 + j * (SR / G);
    };
    // slot and barrier parity of Y1(j)
    auto y1_slot = [](int j) { return L::NY1 == 2 ? j & 1 : 0; };
    auto y1_parity = [](int j) { return uint32_t(L::NY1 == 2 ? (j >> 1) & 1 : j & 1); };

    if (run) {
        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer
            if (lane == 0) {
                const CUtensorMap* mx1 = state_tile ? &map_cx1 : &map_x1;
                const CUtensorMap* mx2 = state_tile ? &map_cx2 : &map_x2;
                mbar_expect_tx(x_full, (PASS == DV ? 1 : 2) * L::RES);
                for (int s = 0; s < SLABS; ++s) {
                    if (PASS == DQ) {
                        tma_load_3d(smem + L::X1 + s * SLAB_RES, mx1, x_full, s * 64, kvh * G, t0);
                        tma_load_3d(smem + L::X2 + s * SLAB_RES, mx2, x_full, s * 64, kvh * G, t0);
                    } else {
                        tma_load_3d(smem + L::X1 + s * SLAB_RES, mx1, x_full, s * 64, kvh, t0);
                        if (PASS == DK) tma_load_3d(smem + L::X2 + s * SLAB_RES, mx2, x_full, s * 64, kvh, t0);
                    }
                }
                // The two streams drain at different times (Y2 right after its score MMA, Y1 after OUT, or the
                // other way round for DV), so each is refilled as soon as its own slot is free.
                const int head0 = PASS == DQ ? kvh : kvh * G;
                int i1 = 0, i2 = 0;
                uint64_t idle_since = 0;
                uint32_t spins = 0;
                while (i1 < n_iter || i2 < n_iter) {
                    bool progressed = false;
                    if (i1 < n_iter && mbar_try_wait(&y1_empty[y1_slot(i1)], y1_parity(i1) ^ 1)) {
                        bool from_state;
                        const int r0 = stream_origin(i1, from_state);
                        const int slot = y1_slot(i1);
                        mbar_expect_tx(&y1_full[slot], L::STR);
                        for (int s = 0; s < SLABS; ++s)
                            tma_load_3d(smem + L::Y1 + slot * L::STR + s * L::SLAB_STR, from_state ? &map_cy1 : &map_y1,
                                        &y1_full[slot], s * 64, head0, r0);
                        ++i1;
                        progressed = true;
                    }
                    if (i2 < n_iter && mbar_try_wait(y2_empty, (i2 & 1) ^ 1)) {
                        bool from_state;
                        const int r0 = stream_origin(i2, from_state);
                        mbar_expect_tx(y2_full, L::STR);
                        for (int s = 0; s < SLABS; ++s)
                            tma_load_3d(smem + L::Y2 + s * L::SLAB_STR, from_state ? &map_cy2 : &map_y2, y2_full, s * 64,
                                        head0, r0);
                        ++i2;
                        progressed = true;
                    }
                    if (progressed) {
                        idle_since = 0;
                        spins = 0;
                    } else {
                        if (ab.raised()) break;
                        if ((++spins & 0x3ff) == 0) {
                            const uint64_t now = global_timer_ns();
                            if (idle_since == 0) idle_since = now;
                            else if (now - idle_since > kWaitBudgetNs) { ab.raise(401); break; }
                        }
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer
            if (lane == 0) {
                constexpr uint32_t idesc_a = instr_desc(ROWS, SR, 1, 1, 0, 0);
                constexpr uint32_t idesc_o = instr_desc(ROWS, D, 1, 1, 0, 1);      // B operand MN-major
                const uint32_t sx1 = smem_u32(smem + L::X1), sx2 = smem_u32(smem + L::X2);
                const uint32_t sy1 = smem_u32(smem + L::Y1), sy2 = smem_u32(smem + L::Y2);
                // Event-driven issue: OUT(jo) goes as soon as E(jo) is in tensor memory, the score MMAs of
                // tile ja as soon as its streamed tiles have landed and its score buffer is free - whichever is
                // ready first, so that a tile still in flight never holds back an MMA whose inputs are there.
                auto ready = [&](uint64_t* bar, uint32_t parity) { return mbar_try_wait(bar, parity); };
                if (mbar_wait(x_full, 0, ab, 406)) {
                    int ja = 0, jo = 0;             // next score tile, next OUT
                    bool a1_done = false;           // A1(ja) issued, A2(ja) still to come
                    uint64_t idle_since = 0;
                    uint32_t spins = 0;
                    while (jo < n_iter) {
                        bool progressed = false;
                        // ---- OUT(jo) += E(jo) * B
                        if (jo < ja && ready(e_full, jo & 1) && (PASS != DV || ready(y2_full, jo & 1))) {
                            tc_fence_after();
                            const uint32_t sb = PASS == DV ? sy2 : sy1 + y1_slot(jo) * L::STR;
#pragma unroll
                            for (int kk = 0; kk < SR / 16; ++kk) {
                                uint64_t db = smem_desc_sw128(sb + kk * 2048, L::SLAB_STR, 1024);
                                mma_bf16_ts(tmem_out, tmem_base + (jo & 1) * SR + kk * 8, db, idesc_o, (jo | kk) != 0);
                            }
                            mma_commit(out_done);
                            if (PASS == DV) mma_commit(y2_empty);
                            else mma_commit(&y1_empty[y1_slot(jo)]);
                            ++jo;
                            progressed = true;
                        }
                        // ---- scores of tile ja into buffer ja & 1
                        if (!progressed && ja < n_iter && ja - jo <= 1) {
                            const int b = ja & 1;
                            if (!a1_done) {
                                // Buffer b fed OUT(ja-2) as its A operand; that MMA must have finished.  It has if
                                // OUT(ja-1) was issued (E(ja-1) is only stored after it); otherwise ask the barrier.
                                const bool buffer_free = ja < 2 || jo == ja || ready(out_done, (jo - 1) & 1);
                                if (buffer_free && ready(&y1_full[y1_slot(ja)], y1_parity(ja))) {
                                    tc_fence_after();
#pragma unroll
                                    for (int s = 0; s < SLABS; ++s)
#pragma unroll
                                        for (int kk = 0; kk < 4; ++kk) {
                                            uint64_t da = smem_desc_sw128(sx1 + s * SLAB_RES + kk * 32, 16, 1024);
                                            uint64_t db = smem_desc_sw128(
                                                sy1 + y1_slot(ja) * L::STR + s * L::SLAB_STR + kk * 32, 16, 1024);
                                            mma_bf16_ss(tmem_base + b * SR, da, db, idesc_a, (s | kk) != 0);
                                        }
                                    progressed = true;
                                    if (PASS == DV) {
                                        mma_commit(&y1_empty[0]);          // Q tile: only the scores read it
                                        mma_commit(&a_full[b]);
                                        ++ja;
                                    } else {
                                        a1_done = true;
                                    }
                                }
                            } else if (ready(y2_full, ja & 1)) {
                                tc_fence_after();
#pragma unroll
                                for (int s = 0; s < SLABS; ++s)
#pragma unroll
                                    for (int kk = 0; kk < 4; ++kk) {
                                        uint64_t da = smem_desc_sw128(sx2 + s * SLAB_RES + kk * 32, 16, 1024);
                                        uint64_t db = smem_desc_sw128(sy2 + s * L::SLAB_STR + kk * 32, 16, 1024);
                                        mma_bf16_ss(tmem_base + 128 + b * SR, da, db, idesc_a, (s | kk) != 0);
                                    }
                                mma_commit(y2_empty);
                                mma_commit(&a_full[b]);
                                a1_done = false;
                                ++ja;
                                progressed = true;
                            }
                        }
                        if (progressed) {
                            idle_since = 0;
                            spins = 0;
                        } else {
                            if (ab.raised()) break;
                            if ((++spins & 0x3ff) == 0) {
                                const uint64_t now = global_timer_ns();
                                if (idle_since == 0) idle_since = now;
                                else if (now - idle_since > kWaitBudgetNs) { ab.raise(407); break; }
                            }
                        }
                    }
                }
            }
        } else {
            // ------------------------------------------------------------ elementwise step + epilogue (warps 2..9)
            // Two warps share a TMEM lane quadrant: warp w reads lanes (w & 3) * 32.., and half h = (w - 2) / 4
            // of the score columns (and of the output columns in the epilogue).
            const int part = warp & 3;
            const int half = (warp - 2) >> 2;
            const int row = part * 32 + lane;                 // TMEM lane = resident row
            const uint32_t lane_addr = uint32_t(part * 32) << 16;
            const float c = p.scale * LOG2E;
            const int tid = threadIdx.x - 64;                 // 0..255 among these warps

            // resident-row facts
            bool lane_valid;
            int lane_key = 0, lane_lo = 0, lane_hi = 0;
            float lane_lse2 = 0.f, lane_delta = 0.f;
            int64_t lane_token = 0;
            int lane_head = 0;
            if (PASS == DQ) {
                const int tok_local = row / G;
                lane_head = kvh * G + row % G;
                lane_valid = tok_local < t1;
                lane_token = int64_t(t0) + tok_local;
                if (lane_valid) {
                    lane_lo = p.row_lo[lane_token];
                    lane_hi = p.row_hi[lane_token];
                    lane_lse2 = p.lse[int64_t(lane_head) * p.tq + lane_token] * LOG2E;
                    lane_delta = p.delta[int64_t(lane_head) * p.tq + lane_token];
                }
            } else {
                lane_valid = row < t1;
                lane_key = t0 + row;
            }

            // facts of the streamed query rows of tile j (DK/DV), fetched one tile ahead
            auto column_facts = [&](int j) {
                ColInfo ci;
                ci.lse2 = 0.f; ci.delta = 0.f; ci.lo = 0; ci.hi = 0;              // lo == hi: sees nothing
                if (PASS != DQ && tid < SR && j < n_iter) {
                    bool unused;
                    const int64_t token = int64_t(stream_origin(j, unused)) + tid / G;
                    const int head = kvh * G + tid % G;
                    if (token < t3) {
                        ci.lse2 = p.lse[int64_t(head) * p.tq + token] * LOG2E;
                        ci.delta = p.delta[int64_t(head) * p.tq + token];
                        if (state_tile) { ci.lo = INT_MIN; ci.hi = INT_MAX; }
                        else { ci.lo = p.row_lo[token]; ci.hi = p.row_hi[token]; }
                    }
                }
                return ci;
            };
            ColInfo next_facts = column_facts(0);
            bool ok = true;     // after a failed wait the loop only keeps the named barrier in step
            for (int j = 0; j < n_iter; ++j) {
                const int b = j & 1;
                bool from_state;
                const int r0 = stream_origin(j, from_state);
                if (PASS != DQ) {
                    if (tid < SR) cols[b * SR + tid] = next_facts;              // shared through shared memory
                    named_barrier(1, EW_WARPS * 32);
                    next_facts = column_facts(j + 1);                           // in flight during this tile's math
                }
                if (ok) ok = mbar_wait(&a_full[b], (j >> 1) & 1, ab, 409);
                float s[HALF], dp[HALF];
                const int c0 = half * HALF;                   // first score column of this warp
                if (ok) {
                    tc_fence_after();
#pragma unroll
                    for (int cc = 0; cc < HALF; cc += 32) {
                        tmem_ld32(tmem_base + lane_addr + b * SR + c0 + cc, reinterpret_cast<uint32_t*>(s + cc));
                        if (PASS != DV)
                            tmem_ld32(tmem_base + lane_addr + 128 + b * SR + c0 + cc,
                                      reinterpret_cast<uint32_t*>(dp + cc));
                    }
                    tmem_wait_ld();
                }
                // E is written over the first half of the score buffer, i.e. over columns the OTHER warp of this
                // lane quadrant reads its scores from: nobody stores before everybody has loaded.
                named_barrier(2, EW_WARPS * 32);
                if (!ok) continue;

                if (PASS == DQ) {
                    const int lo = from_state ? t6 : lane_lo;
                    const int hi = from_state ? t6 + t7 : lane_hi;
#pragma unroll
                    for (int i = 0; i < HALF; ++i) {
                        const int key = r0 + c0 + i;
                        const bool vis = lane_valid && key >= lo && key < hi;
                        const float pr = vis ? fast_exp2(fmaf(s[i], c, -lane_lse2)) : 0.f;
                        s[i] = pr * (dp[i] - lane_delta) * p.scale;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < HALF; ++i) {
                        const ColInfo ci = cols[b * SR + c0 + i];
                        const bool vis = lane_valid && lane_key >= ci.lo && lane_key < ci.hi;
                        const float pr = vis ? fast_exp2(fmaf(s[i], c, -ci.lse2)) : 0.f;
                        s[i] = PASS == DV ? pr : pr * (dp[i] - ci.delta) * p.scale;
                    }
                }

                // E(j) may only be stored once OUT(j-1) has completed (a tcgen05.st while a TS-form MMA reads its
                // A operand from tensor memory corrupts results, whatever the columns).
                if (j > 0) {
                    ok = mbar_wait(out_done, (j - 1) & 1, ab, 410);
                    if (!ok) continue;
                    tc_fence_after();
                }
                // packed bf16 over the first SR / 2 columns of the score buffer: this warp's half of them
                uint32_t w[HALF / 2];
#pragma unroll
                for (int i = 0; i < HALF / 2; ++i) w[i] = pack_bf16(s[2 * i], s[2 * i + 1]);
                if (HALF == 64) tmem_st32(tmem_base + lane_addr + b * SR + half * (HALF / 2), w);
                else tmem_st16(tmem_base + lane_addr + b * SR + half * (HALF / 2), w);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(e_full);
            }

            // epilogue: OUT -> bf16, each warp of a quadrant takes half of the D columns
            if (ok && mbar_wait(out_done, (n_iter - 1) & 1, ab, 411)) {
                tc_fence_after();
                __nv_bfloat16* dst;
                if (PASS == DQ) dst = p.out + (lane_token * p.q_heads + lane_head) * D;
                else dst = (state_tile ? p.out_state : p.out) + (int64_t(lane_key) * p.kv_heads + kvh) * D;
#pragma unroll 1
                for (int cc = half * (D / 2); cc < (half + 1) * (D / 2); cc += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem_out + lane_addr + cc, o);
                    tmem_wait_ld();
                    if (lane_valid) {
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) {
                            uint4 v;
                            v.x = pack_bf16(__uint_as_float(o[v4 * 8 + 0]), __uint_as_float(o[v4 * 8 + 1]));
                            v.y = pack_bf16(__uint_as_float(o[v4 * 8 + 2]), __uint_as_float(o[v4 * 8 + 3]));
                            v.z = pack_bf16(__uint_as_float(o[v4 * 8 + 4]), __uint_as_float(o[v4 * 8 + 5]));
                            v.w = pack_bf16(__uint_as_float(o[v4 * 8 + 6]), __uint_as_float(o[v4 * 8 + 7]));
                            *reinterpret_cast<uint4*>(dst + cc + v4 * 8) = v;
                        }
                    }
                }
            }
        }
    } else if (warp >= 2 && warp < 6 && n_iter == 0 && !ab.raised()) {
        // no query sees this tile (or the tile has no key): its gradient rows are zero
        const int row = (warp & 3) * 32 + lane;
        if (PASS == DQ) {
            if (row / G < t1) {
                __nv_bfloat16* dst = p.out + ((int64_t(t0) + row / G) * p.q_heads + kvh * G + row % G) * D;
                for (int cc = 0; cc < D; cc += 8) *reinterpret_cast<uint4*>(dst + cc) = make_uint4(0, 0, 0, 0);
            }
        } else if (row < t1) {
            __nv_bfloat16* dst = (state_tile ? p.out_state : p.out) + (int64_t(t0 + row) * p.kv_heads + kvh) * D;
            for (int cc = 0; cc < D; cc += 8) *reinterpret_cast<uint4*>(dst + cc) = make_uint4(0, 0, 0, 0);
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (ab.raised()) {
        uint64_t t_start = global_timer_ns();
        while (global_timer_ns() - t_start < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// delta[head, token] = sum_d dO * O, one warp per (token, head).
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ out, int64_t ldo, const __nv_bfloat16* __restrict__ dout,
                                       int64_t ldd, int64_t hsd, float* __restrict__ delta, int64_t tq, int q_heads,
                                       int d) {
    const int lane = threadIdx.x & 31;
    const int64_t item = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= tq * q_heads) return;
    const int64_t token = item / q_heads;
    const int head = (int)(item % q_heads);
    const __nv_bfloat16* po = out + token * ldo + int64_t(head) * d;
    const __nv_bfloat16* pd = dout + token * ldd + int64_t(head) * hsd;
    float acc = 0.f;
    for (int i = lane * 8; i < d; i += 256) {
        const uint4 a = *reinterpret_cast<const uint4*>(po + i);
        const uint4 b = *reinterpret_cast<const uint4*>(pd + i);
        const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 fa = __bfloat1622float2(ha[e]), fb = __bfloat1622float2(hb[e]);
            acc += fa.x * fb.x + fa.y * fb.y;
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) delta[int64_t(head) * tq + token] = acc;
}

int row_map(CUtensorMap* map, const void* base, int64_t tokens, int heads, int d, int64_t ld, int64_t hs, int box_heads,
            int box_tokens) {
    uint64_t dims[3] = {(uint64_t)d, (uint64_t)heads, (uint64_t)tokens};
    uint64_t strides[2] = {(uint64_t)hs * 2, (uint64_t)ld * 2};
    uint32_t box[3] = {64, (uint32_t)box_heads, (uint32_t)box_tokens};
    return bg_make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int D, int PASS>
int launch_pass(const CUtensorMap* m, const BwdParams& p, int n_tiles, cudaStream_t stream) {
    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_bwd_kernel<D, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Layout<D, PASS>::TOTAL);
        if (e != cudaSuccess) {
            bg_set_error("bg_varlen_attention_backward: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    if (n_tiles == 0) return BG_OK;
    dim3 grid((unsigned)n_tiles, (unsigned)p.kv_heads);
    attention_bwd_kernel<D, PASS><<<grid, THREADS, Layout<D, PASS>::TOTAL, stream>>>(m[0], m[1], m[2], m[3], m[4], m[5],
                                                                                    m[6], m[7], p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        bg_set_error("bg_varlen_attention_backward: launch: %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

}  // namespace

extern "C" int bg_varlen_attention_backward(
    const void* q, int64_t ldq, int64_t hsq, const void* k, const void* v, int64_t ldkv, int64_t hskv, const void* ck,
    const void* cv, int64_t ldc, int64_t hsc, const void* out, const void* dout, int64_t ldd, int64_t hsd,
    const float* lse, float* delta, void* dq, void* dk, void* dv, void* dck, void* dcv, const int32_t* q_tiles,
    int32_t n_q_tiles, const int32_t* kv_tiles, int32_t n_kv_tiles, const int32_t* row_lo, const int32_t* row_hi,
    int64_t tq, int64_t tk, int64_t ts, int q_heads, int kv_heads, int head_dim, float scale, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (tq < 0 || tk <= 0 || n_q_tiles < 0 || n_kv_tiles < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) {
        bg_set_error("bg_varlen_attention_backward: bad shape");
        return BG_ERR_SHAPE;
    }
    const int g = q_heads / kv_heads;
    if ((g != 1 && g != 2 && g != 4 && g != 8) || (head_dim != 64 && head_dim != 256)) {
        bg_set_error("bg_varlen_attention_backward: supports head_dim 64 or 256 and a GQA group of 1, 2, 4 or 8 "
                     "(got head_dim %d, group %d)", head_dim, g);
        return BG_ERR_SHAPE;
    }
    if (ldq % 8 || ldkv % 8 || hsq % 8 || hskv % 8 || ldd % 8 || hsd % 8 || (ck && (ldc % 8 || hsc % 8)) ||
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
          reinterpret_cast<uintptr_t>(ck) | reinterpret_cast<uintptr_t>(cv) | reinterpret_cast<uintptr_t>(out) |
          reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
          reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(dck) | reinterpret_cast<uintptr_t>(dcv)) & 15)) {
        bg_set_error("bg_varlen_attention_backward: pointers must be 16-byte aligned and strides multiples of 8 elements");
        return BG_ERR_ALIGN;
    }
    if ((ck != nullptr) != (dck != nullptr) || (cv != nullptr) != (dcv != nullptr) || (ck != nullptr) != (cv != nullptr)) {
        bg_set_error("bg_varlen_attention_backward: state keys, values and their gradients come together");
        return BG_ERR_SHAPE;
    }
    if (tq == 0) return BG_OK;

    // delta = rowsum(dO * O)
    {
        const int64_t items = tq * q_heads;
        attention_delta_kernel<<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(out), (int64_t)q_heads * head_dim, static_cast<const __nv_bfloat16*>(dout),
            ldd, hsd, delta, tq, q_heads, head_dim);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            bg_set_error("bg_varlen_attention_backward: launch(delta): %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
    }

    BwdParams p;
    p.row_lo = row_lo; p.row_hi = row_hi; p.lse = lse; p.delta = delta; p.tq = tq;
    p.q_heads = q_heads; p.kv_heads = kv_heads; p.scale = scale;
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;

    // Tensor maps.  Query-type tiles are (token, head-in-group) rows; key-type tiles are keys of one KV head.
    constexpr int STREAM = 64;     // streamed rows of the DQ and DK passes; DV streams ROWS-row tiles (the *_res boxes)
    CUtensorMap q_res, do_res, q_str, do_str, k_res, v_res, k_str, v_str, ck_res, cv_res, ck_str, cv_str;
    int rc = row_map(&q_res, q, tq, q_heads, head_dim, ldq, hsq, g, ROWS / g);
    if (!rc) rc = row_map(&do_res, dout, tq, q_heads, head_dim, ldd, hsd, g, ROWS / g);
    if (!rc) rc = row_map(&q_str, q, tq, q_heads, head_dim, ldq, hsq, g, STREAM / g);
    if (!rc) rc = row_map(&do_str, dout, tq, q_heads, head_dim, ldd, hsd, g, STREAM / g);
    if (!rc) rc = row_map(&k_res, k, tk, kv_heads, head_dim, ldkv, hskv, 1, ROWS);
    if (!rc) rc = row_map(&v_res, v, tk, kv_heads, head_dim, ldkv, hskv, 1, ROWS);
    if (!rc) rc = row_map(&k_str, k, tk, kv_heads, head_dim, ldkv, hskv, 1, STREAM);
    if (!rc) rc = row_map(&v_str, v, tk, kv_heads, head_dim, ldkv, hskv, 1, STREAM);
    if (rc) return rc;
    if (ck) {
        rc = row_map(&ck_res, ck, ts, kv_heads, head_dim, ldc, hsc, 1, ROWS);
        if (!rc) rc = row_map(&cv_res, cv, ts, kv_heads, head_dim, ldc, hsc, 1, ROWS);
        if (!rc) rc = row_map(&ck_str, ck, ts, kv_heads, head_dim, ldc, hsc, 1, STREAM);
        if (!rc) rc = row_map(&cv_str, cv, ts, kv_heads, head_dim, ldc, hsc, 1, STREAM);
        if (rc) return rc;
    } else {
        ck_res = k_res; cv_res = v_res; ck_str = k_str; cv_str = v_str;
    }

    // DQ: resident Q, dO; streamed K, V (state K, V first)
    {
        const CUtensorMap m[8] = {q_res, do_res, q_res, do_res, k_str, v_str, ck_str, cv_str};
        p.tiles = q_tiles; p.out = static_cast<__nv_bfloat16*>(dq); p.out_state = nullptr;
        rc = head_dim == 64 ? launch_pass<64, DQ>(m, p, n_q_tiles, stream) : launch_pass<256, DQ>(m, p, n_q_tiles, stream);
        if (rc) return rc;
    }
    // DK: resident K, V (or state K, V); streamed Q, dO
    {
        const CUtensorMap m[8] = {k_res, v_res, ck_res, cv_res, q_str, do_str, q_str, do_str};
        p.tiles = kv_tiles; p.out = static_cast<__nv_bfloat16*>(dk); p.out_state = static_cast<__nv_bfloat16*>(dck);
        rc = head_dim == 64 ? launch_pass<64, DK>(m, p, n_kv_tiles, stream) : launch_pass<256, DK>(m, p, n_kv_tiles, stream);
        if (rc) return rc;
        // DV: resident K; streamed Q, dO in 128-row tiles
        const CUtensorMap mv[8] = {k_res, v_res, ck_res, cv_res, q_res, do_res, q_res, do_res};
        p.out = static_cast<__nv_bfloat16*>(dv); p.out_state = static_cast<__nv_bfloat16*>(dcv);
        rc = head_dim == 64 ? launch_pass<64, DV>(mv, p, n_kv_tiles, stream) : launch_pass<256, DV>(mv, p, n_kv_tiles, stream);
        if (rc) return rc;
    }
    return BG_OK;
}
