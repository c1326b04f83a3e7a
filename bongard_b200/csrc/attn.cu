// Packed variable-length attention on tcgen05 tensor cores with TMEM accumulators.
//
// A work item is one query tile for one KV head; one persistent CTA per SM walks its share of the
// items (see item_at).  A query tile is 128 rows: 128/G consecutive packed tokens times the G query
// heads that share the KV head (GQA folded into the M dimension, so K/V tiles are fetched once for
// all of them).  Keys arrive in tiles of 128 through TMA in two phases that share ONE running softmax:
//
//   prefix phase   keys [prefix_start, prefix_start + prefix_len) of a second K/V pair (the
//                  decoder's shared state memory); every row of the tile sees all of them.
//   own phase      keys [own_lo, own_hi) of the packed K/V; row r sees [row_lo[r], row_hi[r]).
//
// This single rule covers the three attention modes of the reference:
//   encoder, global         row range = its segment                (bongard/flash_varlen.py:13-22)
//   encoder, sliding window row range = segment clipped to the bidirectional window
//                                                                  (bongard/packing.py:131-133)
//   decoder, state prefix   prefix = owner's state keys, row range = causal (windowed) part of
//                           its own question                       (bongard/flash_varlen.py:1-8, 61-77)
// A tile whose rows belong to several questions of one owner streams the owner's state once.
//
// Roles, by warpgroup (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer (S = Q K^T, O += P V);
// warps 4-7 = softmax (thread = row); warps 8-11 = output (thread = row).  After start-up the groups
// re-divide the register file (setmaxnreg): a softmax thread holds a row of 128 scores and its packed
// probabilities and gets 240 registers, the control warps 96, the output warps keep 168.
// S is double-buffered in TMEM (2 x 128 columns), O lives in TMEM (D columns).
// The probabilities never leave tensor memory: a softmax thread overwrites the first 64 columns
// of the S buffer it has just read with its row of P as packed bf16 (tcgen05.st), and O += P V is
// issued in the TS form (A = P from TMEM, B = V tile in shared memory, MN-major).  Each iteration
// of this kernel is a latency chain (S ready -> softmax -> P ready -> P.V), and keeping P out of
// shared memory removes the stores, their bank conflicts and the generic-to-async proxy fence
// from that chain.  S(j+1) reuses the buffer that held P(j-1); since
// consecutive MMAs overlap in the tensor pipe, the issuer waits for P.V(j-1) to complete first.
// O is only rescaled when a row's running maximum grows by more than 2^8 (lazy rescale).
//
// Items are pipelined: the barrier phases count key tiles across items, so while item i's output is
// written the producer already loads item i+1's Q and first K/V tiles, the MMA thread computes its
// first S and the softmax warps work on it.  The softmax warps pass an item's row sums to the output
// warps through shared memory (l_full) and go on; the output warps read O out of tensor memory,
// release it (o_free: only the first P.V of item i+1 waits for that) and store the tile through a
// staging buffer with TMA.  Measured per item of 9 key tiles (window 1024): with one CTA per item,
// ~6 300 cycles passed before its first S was complete and ~8 000 after its last P.V was issued
// (read-out, stores, exit, launch of the next CTA) out of ~39 000; pipelined, an item takes ~32 000.
#include "common.cuh"

namespace {

using namespace bg;

constexpr int ROWS = 128;         // query rows per tile (tokens x GQA group)
constexpr int KEYS = 128;         // keys per tile
constexpr int THREADS = 384;      // warpgroup 0: TMA producer (warp 0) and MMA issuer (warp 1); 1: softmax; 2: output
constexpr int REGS_CONTROL = 96;  // registers per thread after the warpgroups have re-divided the register file:
constexpr int REGS_SOFTMAX = 240; //   the softmax threads hold a row of 128 scores and its packed probabilities
constexpr int SLAB = 16384;       // 128 rows x 128 B
constexpr float LAZY_LOG2 = 8.f;  // rescale threshold in log2 units

struct AttnParams {
    const int32_t* tiles;    // [n_tiles][8]: q_start q_count own_lo own_hi lo_max hi_min prefix_start prefix_len
    const int32_t* row_lo;   // [Tq]
    const int32_t* row_hi;   // [Tq]
    __nv_bfloat16* out;      // [Tq, Hq * D]
    float* lse;              // [Hq, Tq] or null
    int64_t tq;
    int q_heads, kv_heads;
    float scale_log2;        // softmax scale * log2(e)
    int32_t* status;
    int n_items;             // tile records x KV heads
};

template <int D>
struct Smem {
    static constexpr int SLABS = D / 64;
    static constexpr int Q = 0;
    static constexpr int K = Q + SLABS * SLAB;
    static constexpr int V = K + SLABS * SLAB;
    static constexpr int STAGE_SLABS = SLABS < 2 ? SLABS : 2;     // output staging: 128 of the head_dim columns at a time
    static constexpr int STAGE = V + SLABS * SLAB;
    static constexpr int BARS = STAGE + STAGE_SLABS * SLAB;
    static constexpr int ROWSUM = BARS + 256;                     // [2][128] floats: row sums and running maxima of an item
    static constexpr int TOTAL = ROWSUM + 1024 + 1024;
};

// One work item: a query tile (a record of the plan) for one KV head.
struct Item {
    int q_start, q_count, own_lo, own_hi, lo_max, hi_min, pre_start, pre_len;
    int n_pre, n_tiles, kvh;
};

// The i-th item of this CTA.  Items are numbered tile-major (the KV heads of one tile side by side) over the
// plan's heaviest-first tile list and dealt to the CTAs in rounds, every other round in reverse order, so that
// each CTA gets one item of every weight band and the light end of one band follows the heavy end of the last.
__host__ __device__ __forceinline__ int item_index(int grid, int cta, int round) {
    return round * grid + ((round & 1) ? grid - 1 - cta : cta);
}
__device__ __forceinline__ bool item_at(const AttnParams& p, int round, Item& im) {
    const int it = item_index(int(gridDim.x), int(blockIdx.x), round);
    if (it >= p.n_items) return false;
    const int tile = it / p.kv_heads;
    const int32_t* t = p.tiles + int64_t(tile) * 8;
    im.q_start = __ldg(t + 0); im.q_count = __ldg(t + 1); im.own_lo = __ldg(t + 2); im.own_hi = __ldg(t + 3);
    im.lo_max = __ldg(t + 4); im.hi_min = __ldg(t + 5); im.pre_start = __ldg(t + 6); im.pre_len = __ldg(t + 7);
    im.n_pre = (im.pre_len + KEYS - 1) / KEYS;
    im.n_tiles = im.n_pre + (im.own_hi - im.own_lo + KEYS - 1) / KEYS;
    im.kvh = it - tile * p.kv_heads;
    return true;
}
// The first item with keys at or after `round` (a record without keys has nothing to compute); false at the end.
__device__ __forceinline__ bool next_item(const AttnParams& p, int& round, Item& im) {
    while (item_at(p, round, im)) {
        if (im.n_tiles > 0) return true;
        ++round;
    }
    return false;
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
varlen_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_ck,
                        const __grid_constant__ CUtensorMap map_cv, const __grid_constant__ CUtensorMap map_o,
                        const AttnParams p) {
    using L = Smem<D>;
    constexpr int SLABS = L::SLABS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = bars + 2;
    uint64_t* v_full = bars + 3;
    uint64_t* v_empty = bars + 4;
    uint64_t* s_full = bars + 5;    // [2]
    uint64_t* p_full = bars + 7;    // 4 warp arrivals: P(j) is in tensor memory
    uint64_t* pv_done = bars + 8;
    uint64_t* q_empty = bars + 9;   // the item's last S has been computed: the Q tile may be replaced
    uint64_t* o_free = bars + 10;   // 4 warp arrivals: the item's O (and row sums) have been read by the output warps
    uint64_t* l_full = bars + 11;   // 4 warp arrivals: the item's row sums are in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};
    const int G = p.q_heads / p.kv_heads;

    // Programmatic dependent launch: wait for the predecessor before the first global read (the tile record);
    // the successor may start its own prologue right away.
    pdl_wait();
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        mbar_init(k_full, 1);
        mbar_init(k_empty, 1);
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        for (int b = 0; b < 2; ++b) mbar_init(&s_full[b], 1);
        mbar_init(p_full, 4);
        mbar_init(pv_done, 1);
        mbar_init(q_empty, 1);
        mbar_init(o_free, 4);
        mbar_init(l_full, 4);
        mbar_fence_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;

    // Every role walks the same list of items.  `g` counts the key tiles of the items before the current one:
    // key tile j of the current item is number g + j of this CTA, and the barrier phases follow that number, so
    // the K, V and S/P hand-over runs on across item boundaries.  `done` counts the items before the current one.
    float* row_l = reinterpret_cast<float*>(smem + L::ROWSUM);
    float* row_m = row_l + ROWS;
    // The three warpgroups re-divide the register file: the softmax threads need far more than the rest.
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_CONTROL));
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            Item im;
            int round = 0;
            uint32_t g = 0, done = 0;
            bool ok = true;
            for (; ok && next_item(p, round, im); ++round, ++done) {
                // the Q tile of the item before has been multiplied for the last time
                if (done > 0 && !mbar_wait_parked(q_empty, (done - 1) & 1, ab, 211)) break;
                mbar_expect_tx(q_full, SLABS * SLAB);
                for (int s = 0; s < SLABS; ++s)
                    tma_load_3d(smem + L::Q + s * SLAB, &map_q, q_full, s * 64, im.kvh * G, im.q_start);
                auto load_k = [&](int j) {
                    if (!ok || !mbar_wait_parked(k_empty, ((g + j) & 1) ^ 1, ab, 201)) { ok = false; return; }
                    const bool pre = j < im.n_pre;
                    const int key0 = pre ? im.pre_start + j * KEYS : im.own_lo + (j - im.n_pre) * KEYS;
                    mbar_expect_tx(k_full, SLABS * SLAB);
                    for (int s = 0; s < SLABS; ++s)
                        tma_load_3d(smem + L::K + s * SLAB, pre ? &map_ck : &map_k, k_full, s * 64, im.kvh, key0);
                };
                auto load_v = [&](int j) {
                    if (!ok || !mbar_wait_parked(v_empty, ((g + j) & 1) ^ 1, ab, 202)) { ok = false; return; }
                    const bool pre = j < im.n_pre;
                    const int key0 = pre ? im.pre_start + j * KEYS : im.own_lo + (j - im.n_pre) * KEYS;
                    mbar_expect_tx(v_full, SLABS * SLAB);
                    for (int s = 0; s < SLABS; ++s)
                        tma_load_3d(smem + L::V + s * SLAB, pre ? &map_cv : &map_v, v_full, s * 64, im.kvh, key0);
                };
                // Issue order follows the order in which the slots drain: S(j) completes before
                // P.V(j-1), so K(j+1) is requested before V(j).
                load_k(0);
                load_v(0);
                if (im.n_tiles > 1) load_k(1);
                for (int j = 1; j < im.n_tiles; ++j) {
                    if (j + 1 < im.n_tiles) load_k(j + 1);
                    load_v(j);
                }
                g += im.n_tiles;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = instr_desc(ROWS, KEYS, 1, 1, 0, 0);
            constexpr uint32_t idesc_o = instr_desc(ROWS, D, 1, 1, 0, 1);   // V is MN-major
            const uint32_t sq = smem_u32(smem + L::Q), sk = smem_u32(smem + L::K);
            const uint32_t sv = smem_u32(smem + L::V);
            bool ok = true;
            // S of key tile number gj.  `first`: the item's first tile (its Q tile has to have arrived); `last`: its
            // last one (afterwards the Q tile may be replaced).
            auto issue_s = [&](uint32_t gj, uint32_t done, bool first, bool last) {
                const int b = gj & 1;
                if (!ok) return;
                if (first && !mbar_wait(q_full, done & 1, ab, 205)) { ok = false; return; }
                if (!mbar_wait(k_full, gj & 1, ab, 203)) { ok = false; return; }
                // Buffer b still holds P(gj-2) as the A operand of P.V(gj-2).  Consecutive MMAs overlap in the
                // tensor pipe, so issue order alone does not protect it: wait for that P.V to finish.  An item's
                // first S is issued after the last P.V of the item before, whose P was only stored once
                // P.V(gj-2) had completed: nothing to wait for (and pv_done may already be a phase further).
                if (!first && gj >= 2 && !mbar_wait(pv_done, gj & 1, ab, 204)) { ok = false; return; }
                tc_fence_after();
#pragma unroll
                for (int s = 0; s < SLABS; ++s)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        uint64_t da = smem_desc_sw128(sq + s * SLAB + kk * 32, 16, 1024);
                        uint64_t db = smem_desc_sw128(sk + s * SLAB + kk * 32, 16, 1024);
                        mma_bf16_ss(tmem_base + b * KEYS, da, db, idesc_s, (s | kk) != 0);
                    }
                mma_commit(&s_full[b]);
                mma_commit(k_empty);
                if (last) mma_commit(q_empty);
            };
            Item im, nx;
            int round = 0;
            uint32_t g = 0, done = 0;
            bool have = next_item(p, round, im);
            if (have) issue_s(0, 0, true, im.n_tiles == 1);
            while (have && ok) {
                int round_nx = round + 1;
                const bool have_nx = next_item(p, round_nx, nx);
                const int n = im.n_tiles;
                for (int j = 0; j < n; ++j) {
                    if (j + 1 < n) issue_s(g + j + 1, done, false, j + 2 == n);
                    if (!ok || !mbar_wait(p_full, (g + j) & 1, ab, 206) || !mbar_wait(v_full, (g + j) & 1, ab, 207)) {
                        ok = false;
                        break;
                    }
                    // the first P.V of an item overwrites O: the epilogue of the item before has to have read it
                    if (j == 0 && done > 0 && !mbar_wait(o_free, (done - 1) & 1, ab, 212)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < KEYS / 16; ++kk) {
                        uint64_t db = smem_desc_sw128(sv + kk * 2048, SLAB, 1024);
                        mma_bf16_ts(tmem_o, tmem_base + ((g + j) & 1) * KEYS + kk * 8, db, idesc_o, (j | kk) != 0);
                    }
                    mma_commit(pv_done);
                    mma_commit(v_empty);
                }
                g += n;
                ++done;
                // The next item's first S follows this item's last P.V into the pipe.  (Issuing it before that P.V,
                // as soon as its tiles had arrived, was slower: the P.V then waits behind it.)
                if (have_nx) issue_s(g, done, true, nx.n_tiles == 1);
                im = nx;
                round = round_nx;
                have = have_nx;
            }
        }
    }
    } else if (warp < 8) {
        // ------------------------------------------------------------ softmax (warps 4..7, thread = row)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
        const int part = warp & 3;
        const int row = part * 32 + lane;
        const int tok_local = row / G;
        const uint32_t lane_addr = uint32_t(part * 32) << 16;
        const float c = p.scale_log2;
        const float lazy = LAZY_LOG2 / c;
        Item im;
        int round = 0;
        uint32_t g = 0, done = 0;
        bool ok = true;
        bool have = next_item(p, round, im);
        // this row's own-key range; the next item's record and range are fetched before the current item's
        // epilogue, so that their latency runs under it
        int rlo = 0, rhi = 0;
        if (have && tok_local < im.q_count) {
            rlo = __ldg(p.row_lo + im.q_start + tok_local);
            rhi = __ldg(p.row_hi + im.q_start + tok_local);
        }
        while (ok && have) {
            const bool row_valid = tok_local < im.q_count;
            const int n_tiles = im.n_tiles, n_pre = im.n_pre, pre_start = im.pre_start, pre_len = im.pre_len;
            float m_ref = -INFINITY, l = 0.f;

            for (int j = 0; j < n_tiles; ++j) {
                const uint32_t gj = g + j;
                const int b = gj & 1;
                if (!mbar_wait(&s_full[b], (gj >> 1) & 1, ab, 208)) { ok = false; break; }
                tc_fence_after();
                float s[KEYS];
#pragma unroll
                for (int cc = 0; cc < KEYS; cc += 32)
                    tmem_ld32(tmem_base + lane_addr + b * KEYS + cc, reinterpret_cast<uint32_t*>(s + cc));
                tmem_wait_ld();

                const bool pre = j < n_pre;
                const int key0 = pre ? pre_start + j * KEYS : im.own_lo + (j - n_pre) * KEYS;
                const int lo = pre ? pre_start : rlo;
                const int hi = pre ? (row_valid ? pre_start + pre_len : pre_start) : rhi;
                const bool need_mask = pre ? (key0 + KEYS > pre_start + pre_len) || !row_valid
                                           : !(key0 >= im.lo_max && key0 + KEYS <= im.hi_min) || !row_valid;
                // The visible keys of a row are one run [first, last) of the tile, and the runs of a warp's rows differ
                // by a few keys only: a 32-key chunk inside every row's run is skipped by the whole warp.  The votes
                // are taken by all 32 lanes (need_mask differs between the rows of a tile that ends early).
                if (__any_sync(0xffffffffu, need_mask)) {
                    const int first = need_mask ? lo - key0 : 0, last = need_mask ? hi - key0 : KEYS;
#pragma unroll
                    for (int cc = 0; cc < KEYS; cc += 32) {
                        if (__all_sync(0xffffffffu, first <= cc && last >= cc + 32)) continue;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (cc + i < first || cc + i >= last) s[cc + i] = -INFINITY;
                    }
                }
                float mx = s[0];
#pragma unroll
                for (int i = 1; i < KEYS; ++i) mx = fmaxf(mx, s[i]);
                const bool grow = mx > m_ref + lazy;   // false while both are -inf
                float alpha = 1.f;
                if (grow) {
                    alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - mx) * c);
                    m_ref = mx;
                    l *= alpha;
                }
                const float shift = (m_ref == -INFINITY) ? 0.f : m_ref * c;
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < KEYS; ++i) {
                    s[i] = fast_exp2(fmaf(s[i], c, -shift));
                    sum += s[i];
                }
                l += sum;

                // P(j) as packed bf16, formed BEFORE the wait below (the empty asm pins the conversions there): after the
                // wait only the two tensor-memory stores remain on the critical path P.V(j-1) -> P(j) -> P.V(j).
                uint32_t w[KEYS / 2];
#pragma unroll
                for (int i = 0; i < KEYS / 2; ++i) w[i] = pack_bf16(s[2 * i], s[2 * i + 1]);
#pragma unroll
                for (int i = 0; i < KEYS / 2; ++i) asm volatile("" : "+r"(w[i]));
                // P(j) may only be stored once the P.V before it has completed (for an item's first tile that is the
                // last P.V of the item before): a tcgen05.st into tensor memory while a TS-form MMA is still
                // reading its A operand from tensor memory corrupted results on B200, even though the two touch
                // different columns.  The same wait makes O stable for a rescale.
                if (gj > 0) {
                    if (!mbar_wait(pv_done, (gj - 1) & 1, ab, 209)) { ok = false; break; }
                    tc_fence_after();
                    if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                        for (int cc = 0; cc < D; cc += 32) {
                            uint32_t o[32];
                            tmem_ld32(tmem_o + lane_addr + cc, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(tmem_o + lane_addr + cc, o);
                        }
                        tmem_wait_st();
                    }
                }
                // over the first 64 columns of the S buffer this thread has just read
                tmem_st32(tmem_base + lane_addr + b * KEYS, w);
                tmem_st32(tmem_base + lane_addr + b * KEYS + 32, w + 32);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
            }
            if (!ok) break;

            // Hand the row sums to the output warps.  The one buffer is free once they have read the item before.
            if (done > 0 && !mbar_wait(o_free, (done - 1) & 1, ab, 213)) break;
            row_l[row] = l;
            row_m[row] = m_ref;
            __syncwarp();
            if (lane == 0) mbar_arrive(l_full);

            g += n_tiles;
            ++done;
            ++round;
            have = next_item(p, round, im);
            rlo = rhi = 0;
            if (have && tok_local < im.q_count) {
                rlo = __ldg(p.row_lo + im.q_start + tok_local);
                rhi = __ldg(p.row_hi + im.q_start + tok_local);
            }
        }
    } else {
        // ------------------------------------------------------------ output (warps 8..11, thread = row)
        // O / l -> bf16 while the softmax warps are already at work on the next item.  O is released to that
        // item's first P.V as soon as its last columns are in registers.  A full tile leaves through a staging
        // buffer, 128 head_dim columns at a time: every thread writes its row in the 128-byte-swizzled layout and
        // one thread issues a TMA store per 64-column slab - whole cache lines instead of 32 rows x 16 bytes per
        // store instruction.  A tile that ends early (last tile of a run) is stored from registers, since a TMA
        // store would also write the rows past its end.
        const int part = warp & 3;
        const int row = part * 32 + lane;
        const int tok_local = row / G;
        const uint32_t lane_addr = uint32_t(part * 32) << 16;
        const float c = p.scale_log2;
        const bool storer = warp == 8 && lane == 0;
        uint8_t* srow = smem + L::STAGE + row * 128;
        Item im;
        int round = 0;
        uint32_t g = 0, done = 0;
        for (; next_item(p, round, im); ++round, ++done) {
            const int head = im.kvh * G + row % G;
            const bool row_valid = tok_local < im.q_count;
            const int64_t token = int64_t(im.q_start) + tok_local;
            // one decision for the four warps: the named barriers below are not bounded waits
            const bool ready = mbar_wait(l_full, done & 1, ab, 214) && mbar_wait(pv_done, (g + im.n_tiles - 1) & 1, ab, 210);
            if (!named_barrier_all(1, 128, ready)) break;
            tc_fence_after();
            const float l = row_l[row], m_ref = row_m[row];
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = p.out + (token * p.q_heads + head) * D;
            const bool staged = im.q_count == ROWS / G;      // the same for every thread of the CTA
            // a tensor-memory load takes some hundred cycles to return: up to four are in flight per wait
            constexpr int EP = D < 128 ? D : 128;
#pragma unroll 1
            for (int half = 0; half < D; half += EP) {
                uint32_t o[EP];
#pragma unroll
                for (int cc = 0; cc < EP; cc += 32) tmem_ld32(tmem_o + lane_addr + half + cc, o + cc);
                tmem_wait_ld();
                if (half + EP >= D) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_free);
                }
                if (staged) {
                    // the staging buffer is free once the stores issued from it have read it
                    if (storer) tma_store_wait_read();
                    named_barrier(1, 128);
                }
#pragma unroll
                for (int v4 = 0; v4 < EP / 8; ++v4) {
                    uint4 v;
                    v.x = pack_bf16(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                    v.y = pack_bf16(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                    v.z = pack_bf16(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                    v.w = pack_bf16(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                    if (staged) {
                        const int col = v4 * 8;                  // column inside this pass
                        const int chunk = (col & 63) >> 3;       // 16-byte chunk inside the 128-byte slab row
                        *reinterpret_cast<uint4*>(srow + (col >> 6) * SLAB + ((chunk ^ (row & 7)) << 4)) = v;
                    } else if (row_valid) {
                        *reinterpret_cast<uint4*>(dst + half + v4 * 8) = v;
                    }
                }
                if (staged) {
                    fence_async_proxy();
                    named_barrier(1, 128);
                    if (storer) {
                        for (int sl = 0; sl < EP / 64; ++sl)
                            tma_store_3d(&map_o, smem + L::STAGE + sl * SLAB, half + sl * 64, im.kvh * G, im.q_start);
                        tma_store_commit();
                    }
                }
            }
            if (p.lse != nullptr && row_valid) {
                const float ln2 = 0.6931471805599453f;
                p.lse[int64_t(head) * p.tq + token] =
                    l > 0.f ? (m_ref * c + log2f(l)) * ln2 : -INFINITY;
            }
            g += im.n_tiles;
        }
        // the last stores have to have read the staging buffer before the CTA gives up its shared memory
        if (storer) tma_store_wait_read();
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

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mck,
           const CUtensorMap& mcv, const CUtensorMap& mo, const AttnParams& p, cudaStream_t stream) {
    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(varlen_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Smem<D>::TOTAL);
        if (e != cudaSuccess) {
            bg_set_error("bg_varlen_attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    const int sms = bg_num_sms();       // one CTA per SM (shared and tensor memory are used in full)
    dim3 grid((unsigned)(p.n_items < sms ? p.n_items : sms));
    cudaError_t e = launch_kernel(varlen_attention_kernel<D>, grid, dim3(THREADS), Smem<D>::TOTAL, stream, 0, mq, mk, mv,
                                  mck, mcv, mo, p);
    if (e != cudaSuccess) {
        bg_set_error("bg_varlen_attention: launch: %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}

int kv_map(CUtensorMap* map, const void* base, int64_t tokens, int heads, int d, int64_t ld, int64_t hs) {
    uint64_t dims[3] = {(uint64_t)d, (uint64_t)heads, (uint64_t)tokens};
    uint64_t strides[2] = {(uint64_t)hs * 2, (uint64_t)ld * 2};
    uint32_t box[3] = {64, 1, KEYS};
    return bg_make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

// Which work item (tile record * kv_heads + KV head) CTA `cta` of a grid of `grid` persistent CTAs takes in its
// `round`-th turn; the CTA is done at the first index that is not below tile records x KV heads.  Host-side
// mirror of the kernel's dealing rule, for tests and for callers that want to predict the balance of a plan.
extern "C" int bg_attention_item_index(int grid, int cta, int round) {
    return (grid <= 0 || cta < 0 || cta >= grid || round < 0) ? -1 : item_index(grid, cta, round);
}

// Query rows one tile of bg_varlen_attention covers (128 for every supported head size).
// A tile record may hold up to this many rows / (q_heads / kv_heads) consecutive tokens.
extern "C" int bg_attention_tile_rows(int head_dim) { (void)head_dim; return 128; }

extern "C" int bg_varlen_attention(const void* q, int64_t ldq, int64_t hsq, const void* k, const void* v,
                                   int64_t ldkv, int64_t hskv, const void* ck, const void* cv, int64_t ldc,
                                   int64_t hsc, void* out, float* lse,
                                   const int32_t* tiles, int32_t n_tiles, const int32_t* row_lo,
                                   const int32_t* row_hi, int64_t tq, int64_t tk, int64_t ts, int q_heads,
                                   int kv_heads, int head_dim, float scale, void* stream) {
    if (tq < 0 || tk <= 0 || n_tiles < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) {
        bg_set_error("bg_varlen_attention: bad shape");
        return BG_ERR_SHAPE;
    }
    const int g = q_heads / kv_heads;
    if ((g != 1 && g != 2 && g != 4 && g != 8) || (head_dim != 64 && head_dim != 256)) {
        bg_set_error("bg_varlen_attention: supports head_dim 64 or 256 and a GQA group of 1, 2, 4 or 8 "
                     "(got head_dim %d, group %d)", head_dim, g);
        return BG_ERR_SHAPE;
    }
    if (ldq % 8 || ldkv % 8 || hsq % 8 || hskv % 8 || (ck && (ldc % 8 || hsc % 8)) ||
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
          reinterpret_cast<uintptr_t>(ck) | reinterpret_cast<uintptr_t>(cv) | reinterpret_cast<uintptr_t>(out)) & 15)) {
        bg_set_error("bg_varlen_attention: pointers must be 16-byte aligned and strides multiples of 8 elements");
        return BG_ERR_ALIGN;
    }
    if (n_tiles == 0 || tq == 0) return BG_OK;

    CUtensorMap mq, mk, mv, mck, mcv;
    {
        uint64_t dims[3] = {(uint64_t)head_dim, (uint64_t)q_heads, (uint64_t)tq};
        uint64_t strides[2] = {(uint64_t)hsq * 2, (uint64_t)ldq * 2};
        uint32_t box[3] = {64, (uint32_t)g, (uint32_t)(ROWS / g)};
        int rc = bg_make_tensor_map(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, q, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    int rc = kv_map(&mk, k, tk, kv_heads, head_dim, ldkv, hskv);
    if (!rc) rc = kv_map(&mv, v, tk, kv_heads, head_dim, ldkv, hskv);
    if (!rc && ck) rc = kv_map(&mck, ck, ts, kv_heads, head_dim, ldc, hsc);
    if (!rc && cv) rc = kv_map(&mcv, cv, ts, kv_heads, head_dim, ldc, hsc);
    if (rc) return rc;
    if (!ck) { mck = mk; mcv = mv; }
    CUtensorMap mo;      // the output [tq, q_heads, head_dim], stored in the boxes the Q tiles are loaded in
    {
        uint64_t dims[3] = {(uint64_t)head_dim, (uint64_t)q_heads, (uint64_t)tq};
        uint64_t strides[2] = {(uint64_t)head_dim * 2, (uint64_t)q_heads * head_dim * 2};
        uint32_t box[3] = {64, (uint32_t)g, (uint32_t)(ROWS / g)};
        rc = bg_make_tensor_map(&mo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }

    AttnParams p;
    p.tiles = tiles; p.row_lo = row_lo; p.row_hi = row_hi;
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse; p.tq = tq;
    p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;
    p.n_items = n_tiles * kv_heads;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return head_dim == 64 ? launch<64>(mq, mk, mv, mck, mcv, mo, p, s) : launch<256>(mq, mk, mv, mck, mcv, mo, p, s);
}
