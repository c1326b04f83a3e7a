// Packed variable-length attention for head_dim 256 on CTA PAIRS (cluster of 2, tcgen05 cta_group::2).
//
// Same contract as the single-CTA kernel in attn.cu - query tiles, a prefix phase (the decoder's
// shared state) and an own phase with per-row key ranges under ONE running softmax - but a tile
// record now covers 256 query rows (2 x 128/G tokens x G query heads of one KV head) and a pair of
// CTAs works on it together, each CTA on its own 128 rows:
//
//   S = Q K^T    one MMA per 16 of head_dim with M = 256, N = 128 keys.  A = each CTA's own Q tile
//                (shared memory); the B operand is split along N, so a CTA loads only 64 of the
//                128 keys of a tile (32 KB instead of 64 KB).
//   O += P V     M = 256, N = 256 head_dim columns, K = 128 keys.  A = each CTA's own P, read from
//                tensor memory (TS form); B is split along N, so a CTA loads all 128 keys but only
//                128 of V's 256 columns (32 KB instead of 64 KB).
//
// At head_dim 256 a 128-row tile needs 128 KB of K and V per 128 keys against 2048 tensor-core
// cycles of work, i.e. 64 B per cycle and SM out of L2, which the single-CTA kernel cannot get (it
// runs at the L2-to-SM rate).  The pair halves that stream per SM, and the halved tiles leave room
// for TWO K slots and TWO V slots beside the resident Q tile, so the next tile is on its way while
// the current one is being multiplied.  Everything else is as in attn.cu: S double-buffered in
// tensor memory, P written as packed bf16 over the S buffer it came from, lazy rescaling of O.
//
// Barriers sit at the same offset in both CTAs.  Used in the leader (rank 0) only, credited by both
// CTAs: q_full, k_full[], v_full[] (TMA bytes), p_full (8 warp arrivals).  One per CTA, signalled by
// the leader's MMA thread with one commit per CTA: s_full[], k_empty[], v_empty[], pv_done.
// Every TMA load has one destination: each CTA fetches its own halves.
#include "common.cuh"

namespace {

using namespace bg;

constexpr int D = 256;
constexpr int ROWS = 128;              // query rows per CTA
constexpr int KEYS = 128;              // keys per tile
constexpr int THREADS = 192;
constexpr int SLAB = 16384;            // 128 rows x 128 B
constexpr int HSLAB = 8192;            //  64 rows x 128 B
constexpr int Q_BYTES = 4 * SLAB;      // 128 rows x 256 head_dim
constexpr int K_STAGE = 4 * HSLAB;     //  64 keys x 256 head_dim
constexpr int V_STAGE = 2 * SLAB;      // 128 keys x 128 head_dim columns
constexpr int NK = 2, NV = 2;
constexpr float LAZY_LOG2 = 8.f;

struct PairAttnParams {
    const int32_t* tiles;    // [n_tiles][8]: q_start q_count own_lo own_hi lo_max hi_min prefix_start prefix_len
    const int32_t* row_lo;   // [Tq]
    const int32_t* row_hi;   // [Tq]
    __nv_bfloat16* out;      // [Tq, Hq * D]
    float* lse;              // [Hq, Tq] or null
    int64_t tq;
    int q_heads, kv_heads;
    float scale_log2;
    int32_t* status;
};

struct L {
    static constexpr int Q = 0;
    static constexpr int K = Q + Q_BYTES;
    static constexpr int V = K + NK * K_STAGE;
    static constexpr int BARS = V + NV * V_STAGE;
    static constexpr int TOTAL = BARS + 256 + 1024;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
varlen_attention_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_ck,
                             const __grid_constant__ CUtensorMap map_cv, const __grid_constant__ CUtensorMap map_o,
                             const PairAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;              // [NK]
    uint64_t* v_full = k_full + NK;           // [NV]
    uint64_t* k_empty = v_full + NV;          // [NK]
    uint64_t* v_empty = k_empty + NK;         // [NV]
    uint64_t* s_full = v_empty + NV;          // [2]
    uint64_t* p_full = s_full + 2;
    uint64_t* pv_done = p_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const Abort ab{abort_flag, p.status};
    const int kvh = blockIdx.y;
    const int G = p.q_heads / p.kv_heads;
    const int TQ = ROWS / G;                  // tokens per CTA

    // The tile record (and, below, the rows' key ranges) are requested before the barriers are set up and the
    // cluster has synchronised, so that their latency runs under that set-up instead of after it.
    pdl_wait();
    pdl_launch_dependents();
    const int32_t* t = p.tiles + int64_t(blockIdx.x >> 1) * 8;
    const int q_start = t[0], q_count = t[1], own_lo = t[2], own_hi = t[3], lo_max = t[4], hi_min = t[5];
    const int pre_start = t[6], pre_len = t[7];
    const int n_pre = (pre_len + KEYS - 1) / KEYS;
    const int n_own = (own_hi - own_lo + KEYS - 1) / KEYS;
    const int n_tiles = n_pre + n_own;
    const int my_start = q_start + int(rank) * TQ;               // first token of this CTA's rows
    const int my_count = max(0, min(TQ, q_count - int(rank) * TQ));

    // softmax threads: this row's own-key range
    int rlo = 0, rhi = 0;
    if (warp >= 2) {
        const int tok_local = ((warp & 3) * 32 + lane) / G;
        if (tok_local < my_count) {
            rlo = __ldg(p.row_lo + my_start + tok_local);
            rhi = __ldg(p.row_hi + my_start + tok_local);
        }
    }

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < NK; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        for (int s = 0; s < NV; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) mbar_init(&s_full[b], 1);
        mbar_init(p_full, 8);
        mbar_init(pv_done, 1);
        mbar_fence_init();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();               // both CTAs' barriers exist before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;

    if (n_tiles > 0) {
        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer (one per CTA)
            if (lane == 0) {
                const uint32_t lead_q = map_to_cta(smem_u32(q_full), 0);
                if (leader) mbar_expect_tx(q_full, 2 * Q_BYTES);
                for (int s = 0; s < 4; ++s)
                    tma_load_3d_pair(smem + L::Q + s * SLAB, &map_q, lead_q, s * 64, kvh * G, my_start);
                auto load_k = [&](int j) {
                    const int st = j % NK;
                    if (!mbar_wait_parked(&k_empty[st], ((j / NK) & 1) ^ 1, ab, 221)) return;
                    const bool pre = j < n_pre;
                    const int key0 = (pre ? pre_start + j * KEYS : own_lo + (j - n_pre) * KEYS) + int(rank) * 64;
                    const uint32_t lead = map_to_cta(smem_u32(&k_full[st]), 0);
                    if (leader) mbar_expect_tx(&k_full[st], 2 * K_STAGE);
                    for (int s = 0; s < 4; ++s)
                        tma_load_3d_pair(smem + L::K + st * K_STAGE + s * HSLAB, pre ? &map_ck : &map_k, lead, s * 64, kvh,
                                         key0);
                };
                auto load_v = [&](int j) {
                    const int st = j % NV;
                    if (!mbar_wait_parked(&v_empty[st], ((j / NV) & 1) ^ 1, ab, 222)) return;
                    const bool pre = j < n_pre;
                    const int key0 = pre ? pre_start + j * KEYS : own_lo + (j - n_pre) * KEYS;
                    const uint32_t lead = map_to_cta(smem_u32(&v_full[st]), 0);
                    if (leader) mbar_expect_tx(&v_full[st], 2 * V_STAGE);
                    for (int s = 0; s < 2; ++s)
                        tma_load_3d_pair(smem + L::V + st * V_STAGE + s * SLAB, pre ? &map_cv : &map_v, lead,
                                         (int(rank) * 2 + s) * 64, kvh, key0);
                };
                // Slots drain in the order S(0) S(1) PV(0) S(2) PV(1) ...: request in the same order.
                load_k(0);
                load_v(0);
                if (n_tiles > 1) load_k(1);
                for (int j = 1; j < n_tiles; ++j) {
                    if (j + 1 < n_tiles) load_k(j + 1);
                    load_v(j);
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer (leader CTA only)
            // Issuing an MMA blocks this thread for roughly the time the instruction takes in the tensor pipe,
            // so the barriers the NEXT step needs are tested between the MMAs of the current one (a test costs
            // the thread ~30 cycles it would spend blocked anyway); a step then starts without the ~100 cycles
            // of a barrier wait, and only a barrier that really is late is waited for.
            if (lane == 0 && leader) {
                constexpr uint32_t idesc_s = instr_desc(2 * ROWS, KEYS, 1, 1, 0, 0);
                constexpr uint32_t idesc_o = instr_desc(2 * ROWS, D, 1, 1, 0, 1);   // V is MN-major
                const uint32_t sq = smem_u32(smem + L::Q), sk = smem_u32(smem + L::K), sv = smem_u32(smem + L::V);
                // the barrier block sits at the same offset in both CTAs: one mapa per CTA, then plain offsets
                const uint32_t bars_own = map_to_cta(smem_u32(bars), 0), bars_peer = map_to_cta(smem_u32(bars), 1);
                auto commit_both = [&](uint64_t* bar) {
                    const uint32_t off = smem_u32(bar) - smem_u32(bars);
                    mma_commit_pair(bars_own + off);
                    mma_commit_pair(bars_peer + off);
                };
                auto ensure = [&](bool seen, uint64_t* bar, uint32_t parity, int code) {
                    return seen || mbar_wait(bar, parity, ab, code);
                };
                bool ok = mbar_wait(q_full, 0, ab, 225);
                bool k_seen = false, p_seen = false, v_seen = false;
                // S(j): needs K(j) and, for j >= 2, P.V(j-2) complete (buffer j & 1 holds P(j-2), its A operand).
                // While its MMAs go out, P(j-1) and V(j-1) - what the following P.V needs - are tested for.
                auto issue_s = [&](int j) {
                    const int b = j & 1, st = j % NK;
                    ok = ok && ensure(k_seen, &k_full[st], (j / NK) & 1, 223);
                    ok = ok && (j < 2 || mbar_wait(pv_done, j & 1, ab, 224));
                    if (!ok) return;
                    tc_fence_after();
                    p_seen = v_seen = false;
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            uint64_t da = smem_desc_sw128(sq + s * SLAB + kk * 32, 16, 1024);
                            uint64_t db = smem_desc_sw128(sk + st * K_STAGE + s * HSLAB + kk * 32, 16, 1024);
                            mma_bf16_ss_pair(tmem_base + b * KEYS, da, db, idesc_s, (s | kk) != 0);
                        }
                        if (j >= 1 && s >= 1) {
                            if (!p_seen) p_seen = mbar_try_wait(p_full, (j - 1) & 1);
                            if (!v_seen) v_seen = mbar_try_wait(&v_full[(j - 1) % NV], ((j - 1) / NV) & 1);
                        }
                    }
                    commit_both(&s_full[b]);
                    commit_both(&k_empty[st]);
                };
                if (ok) issue_s(0);
                for (int j = 0; j < n_tiles && ok; ++j) {
                    k_seen = false;
                    if (j + 1 < n_tiles) {
                        k_seen = mbar_try_wait(&k_full[(j + 1) % NK], ((j + 1) / NK) & 1);
                        issue_s(j + 1);
                    } else {
                        p_seen = v_seen = false;
                    }
                    const int st = j % NV;
                    ok = ok && ensure(p_seen, p_full, j & 1, 226) && ensure(v_seen, &v_full[st], (j / NV) & 1, 227);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < KEYS / 16; ++kk) {
                        uint64_t db = smem_desc_sw128(sv + st * V_STAGE + kk * 2048, SLAB, 1024);
                        mma_bf16_ts_pair(tmem_o, tmem_base + (j & 1) * KEYS + kk * 8, db, idesc_o, (j | kk) != 0);
                    }
                    commit_both(pv_done);
                    commit_both(&v_empty[st]);
                }
            }
        } else {
            // ------------------------------------------------------------ softmax + epilogue (warps 2..5), own 128 rows
            const int part = warp & 3;
            const int row = part * 32 + lane;
            const int tok_local = row / G;
            const int head = kvh * G + row % G;
            const bool row_valid = tok_local < my_count;
            const int64_t token = int64_t(my_start) + tok_local;
            const uint32_t lane_addr = uint32_t(part * 32) << 16;
            const float c = p.scale_log2;
            const float lazy = LAZY_LOG2 / c;
            float m_ref = -INFINITY, l = 0.f;

            for (int j = 0; j < n_tiles; ++j) {
                const int b = j & 1;
                if (!mbar_wait(&s_full[b], (j >> 1) & 1, ab, 228)) break;
                tc_fence_after();
                float s[KEYS];
#pragma unroll
                for (int cc = 0; cc < KEYS; cc += 32)
                    tmem_ld32(tmem_base + lane_addr + b * KEYS + cc, reinterpret_cast<uint32_t*>(s + cc));
                tmem_wait_ld();

                const bool pre = j < n_pre;
                const int key0 = pre ? pre_start + j * KEYS : own_lo + (j - n_pre) * KEYS;
                const int lo = pre ? pre_start : rlo;
                const int hi = pre ? (row_valid ? pre_start + pre_len : pre_start) : rhi;
                const bool need_mask = pre ? (key0 + KEYS > pre_start + pre_len) || !row_valid
                                           : !(key0 >= lo_max && key0 + KEYS <= hi_min) || !row_valid;
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < KEYS; ++i) {
                        const int key = key0 + i;
                        if (key < lo || key >= hi) s[i] = -INFINITY;
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
                // P(j) may only be stored once P.V(j-1) has completed (a tcgen05.st while a TS-form MMA reads its A
                // operand from tensor memory corrupts results); the same wait makes O stable for a rescale.
                if (j > 0) {
                    mbar_wait(pv_done, (j - 1) & 1, ab, 229);
                    tc_fence_after();
                    if (__any_sync(0xffffffffu, grow)) {
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
                if (lane == 0) mbar_arrive_leader(p_full);
            }

            // epilogue: O / l -> bf16.  A full tile goes through shared memory: every thread writes its row into
            // the (now idle) Q tile's slabs in the 128-byte-swizzled layout and one thread stores the tile with four
            // TMA stores - 512-byte rows in whole cache lines instead of 32 rows x 16 bytes per store instruction,
            // which took 5000 cycles a tile.  A tile that ends early (last tile of a run) keeps the direct stores,
            // since a TMA store would also write the rows past its end.
            const bool staged = my_count == TQ;          // the same for every thread of the CTA
            const bool finished = mbar_wait(pv_done, (n_tiles - 1) & 1, ab, 230);
            if (finished) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16* dst = p.out + (token * p.q_heads + head) * D;
                uint8_t* srow = smem + L::Q + row * 128;
                // a tensor-memory load takes some hundred cycles to return: four are in flight per wait
#pragma unroll 1
                for (int half = 0; half < D; half += 128) {
                    uint32_t o[128];
#pragma unroll
                    for (int cc = 0; cc < 128; cc += 32) tmem_ld32(tmem_o + lane_addr + half + cc, o + cc);
                    tmem_wait_ld();
#pragma unroll
                    for (int v4 = 0; v4 < 16; ++v4) {
                        uint4 v;
                        v.x = pack_bf16(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                        v.y = pack_bf16(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                        v.z = pack_bf16(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                        v.w = pack_bf16(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                        const int col = half + v4 * 8;               // first of 8 head_dim columns
                        if (staged) {
                            const int chunk = (col & 63) >> 3;       // 16-byte chunk inside the 128-byte slab row
                            *reinterpret_cast<uint4*>(srow + (col >> 6) * SLAB + ((chunk ^ (row & 7)) << 4)) = v;
                        } else if (row_valid) {
                            *reinterpret_cast<uint4*>(dst + col) = v;
                        }
                    }
                }
                if (p.lse != nullptr && row_valid) {
                    const float ln2 = 0.6931471805599453f;
                    p.lse[int64_t(head) * p.tq + token] = l > 0.f ? (m_ref * c + log2f(l)) * ln2 : -INFINITY;
                }
            }
            if (staged) {
                // every softmax thread comes here, also after an abort: the barrier below is not a bounded wait
                fence_async_proxy();
                named_barrier(1, 128);
                if (warp == 2 && lane == 0 && !ab.raised()) {
                    for (int s = 0; s < 4; ++s) tma_store_3d(&map_o, smem + L::Q + s * SLAB, s * 64, kvh * G, my_start);
                    tma_store_commit();
                    tma_store_wait_read();
                }
            }
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
    cluster_sync();               // the leader's MMAs read the peer's shared and tensor memory: leave together
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

int kv_map(CUtensorMap* map, const void* base, int64_t tokens, int heads, int64_t ld, int64_t hs, uint32_t box_keys) {
    uint64_t dims[3] = {(uint64_t)D, (uint64_t)heads, (uint64_t)tokens};
    uint64_t strides[2] = {(uint64_t)hs * 2, (uint64_t)ld * 2};
    uint32_t box[3] = {64, 1, box_keys};
    return bg_make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box,
                              CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

// Query rows one tile record of bg_varlen_attention_pair covers: 256 for head_dim 256, 0 (no pair kernel) otherwise.
extern "C" int bg_attention_pair_tile_rows(int head_dim) { return head_dim == D ? 2 * ROWS : 0; }

// bg_varlen_attention for head_dim 256 with tile records of 256 query rows (2 x 128 / group tokens), served
// by CTA pairs.  Arguments, results and error behaviour are those of bg_varlen_attention.
extern "C" int bg_varlen_attention_pair(const void* q, int64_t ldq, int64_t hsq, const void* k, const void* v,
                                        int64_t ldkv, int64_t hskv, const void* ck, const void* cv, int64_t ldc,
                                        int64_t hsc, void* out, float* lse, const int32_t* tiles, int32_t n_tiles,
                                        const int32_t* row_lo, const int32_t* row_hi, int64_t tq, int64_t tk,
                                        int64_t ts, int q_heads, int kv_heads, int head_dim, float scale,
                                        void* stream) {
    if (tq < 0 || tk <= 0 || n_tiles < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) {
        bg_set_error("bg_varlen_attention_pair: bad shape");
        return BG_ERR_SHAPE;
    }
    const int g = q_heads / kv_heads;
    if ((g != 1 && g != 2 && g != 4 && g != 8) || head_dim != D) {
        bg_set_error("bg_varlen_attention_pair: supports head_dim 256 and a GQA group of 1, 2, 4 or 8 "
                     "(got head_dim %d, group %d)", head_dim, g);
        return BG_ERR_SHAPE;
    }
    if (ldq % 8 || ldkv % 8 || hsq % 8 || hskv % 8 || (ck && (ldc % 8 || hsc % 8)) ||
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
          reinterpret_cast<uintptr_t>(ck) | reinterpret_cast<uintptr_t>(cv) | reinterpret_cast<uintptr_t>(out)) & 15)) {
        bg_set_error("bg_varlen_attention_pair: pointers must be 16-byte aligned and strides multiples of 8 elements");
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
    int rc = kv_map(&mk, k, tk, kv_heads, ldkv, hskv, 64);
    if (!rc) rc = kv_map(&mv, v, tk, kv_heads, ldkv, hskv, KEYS);
    if (!rc && ck) rc = kv_map(&mck, ck, ts, kv_heads, ldc, hsc, 64);
    if (!rc && cv) rc = kv_map(&mcv, cv, ts, kv_heads, ldc, hsc, KEYS);
    if (rc) return rc;
    if (!ck) { mck = mk; mcv = mv; }
    CUtensorMap mo;
    {
        uint64_t dims[3] = {(uint64_t)head_dim, (uint64_t)q_heads, (uint64_t)tq};
        uint64_t strides[2] = {(uint64_t)head_dim * 2, (uint64_t)q_heads * head_dim * 2};
        uint32_t box[3] = {64, (uint32_t)g, (uint32_t)(ROWS / g)};
        rc = bg_make_tensor_map(&mo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }

    PairAttnParams p;
    p.tiles = tiles; p.row_lo = row_lo; p.row_hi = row_hi;
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse; p.tq = tq;
    p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;

    static bool configured_on[kBgMaxDevices] = {};
    bool& configured = configured_on[bg_device_slot()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(varlen_attention_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             L::TOTAL);
        if (e != cudaSuccess) {
            bg_set_error("bg_varlen_attention_pair: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            return BG_ERR_LAUNCH;
        }
        configured = true;
    }
    dim3 grid((unsigned)n_tiles * 2, (unsigned)kv_heads);
    cudaError_t e = launch_kernel(varlen_attention_pair_kernel, grid, dim3(THREADS), L::TOTAL,
                                  static_cast<cudaStream_t>(stream), 0, mq, mk, mv, mck, mcv, mo, p);
    if (e != cudaSuccess) {
        bg_set_error("bg_varlen_attention_pair: launch: %s", cudaGetErrorString(e));
        return BG_ERR_LAUNCH;
    }
    return BG_OK;
}
