// Packed variable-length attention on tcgen05 tensor cores with TMEM accumulators.
//
// One CTA computes one query tile for one KV head.  A query tile is 128 rows: 128/G
// consecutive packed tokens times the G query heads that share the KV head (GQA folded
// into the M dimension, so K/V tiles are fetched once for all of them).  Keys arrive in
// tiles of 128 through TMA in two phases that share ONE running softmax:
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
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer (S = Q K^T, O += P V), warps 2-5 = softmax
// (thread = row).  S is double-buffered in TMEM (2 x 128 columns), O lives in TMEM (D columns).
// The probabilities never leave tensor memory: a softmax thread overwrites the first 64 columns
// of the S buffer it has just read with its row of P as packed bf16 (tcgen05.st), and O += P V is
// issued in the TS form (A = P from TMEM, B = V tile in shared memory, MN-major).  Each iteration
// of this kernel is a latency chain (S ready -> softmax -> P ready -> P.V), and keeping P out of
// shared memory removes the stores, their bank conflicts and the generic-to-async proxy fence
// from that chain.  S(j+1) reuses the buffer that held P(j-1); since
// consecutive MMAs overlap in the tensor pipe, the issuer waits for P.V(j-1) to complete first.
// O is only rescaled when a row's running maximum grows by more than 2^8 (lazy rescale).
#include "common.cuh"

namespace {

using namespace bg;

constexpr int ROWS = 128;         // query rows per tile (tokens x GQA group)
constexpr int KEYS = 128;         // keys per tile
constexpr int THREADS = 192;
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
};

template <int D>
struct Smem {
    static constexpr int SLABS = D / 64;
    static constexpr int Q = 0;
    static constexpr int K = Q + SLABS * SLAB;
    static constexpr int V = K + SLABS * SLAB;
    static constexpr int BARS = V + SLABS * SLAB;
    static constexpr int TOTAL = BARS + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
varlen_attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_ck,
                        const __grid_constant__ CUtensorMap map_cv, const AttnParams p) {
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
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Abort ab{abort_flag, p.status};
    const int kvh = blockIdx.y;
    const int G = p.q_heads / p.kv_heads;

    // Programmatic dependent launch: wait for the predecessor before the first global read (the tile record);
    // the successor may start its own prologue right away.
    pdl_wait();
    pdl_launch_dependents();
    const int32_t* t = p.tiles + int64_t(blockIdx.x) * 8;
    const int q_start = t[0], q_count = t[1], own_lo = t[2], own_hi = t[3], lo_max = t[4], hi_min = t[5];
    const int pre_start = t[6], pre_len = t[7];
    const int n_pre = (pre_len + KEYS - 1) / KEYS;
    const int n_own = (own_hi - own_lo + KEYS - 1) / KEYS;
    const int n_tiles = n_pre + n_own;

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

    if (n_tiles > 0) {
        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer
            if (lane == 0) {
                mbar_expect_tx(q_full, SLABS * SLAB);
                for (int s = 0; s < SLABS; ++s)
                    tma_load_3d(smem + L::Q + s * SLAB, &map_q, q_full, s * 64, kvh * G, q_start);
                auto load_k = [&](int j) {
                    if (!mbar_wait_parked(k_empty, (j & 1) ^ 1, ab, 201)) return;
                    const bool pre = j < n_pre;
                    const int key0 = pre ? pre_start + j * KEYS : own_lo + (j - n_pre) * KEYS;
                    mbar_expect_tx(k_full, SLABS * SLAB);
                    for (int s = 0; s < SLABS; ++s)
                        tma_load_3d(smem + L::K + s * SLAB, pre ? &map_ck : &map_k, k_full, s * 64, kvh, key0);
                };
                auto load_v = [&](int j) {
                    if (!mbar_wait_parked(v_empty, (j & 1) ^ 1, ab, 202)) return;
                    const bool pre = j < n_pre;
                    const int key0 = pre ? pre_start + j * KEYS : own_lo + (j - n_pre) * KEYS;
                    mbar_expect_tx(v_full, SLABS * SLAB);
                    for (int s = 0; s < SLABS; ++s)
                        tma_load_3d(smem + L::V + s * SLAB, pre ? &map_cv : &map_v, v_full, s * 64, kvh, key0);
                };
                // Issue order follows the order in which the slots drain: S(j) completes before
                // P.V(j-1), so K(j+1) is requested before V(j).
                load_k(0);
                load_v(0);
                if (n_tiles > 1) load_k(1);
                for (int j = 1; j < n_tiles; ++j) {
                    if (j + 1 < n_tiles) load_k(j + 1);
                    load_v(j);
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer
            if (lane == 0) {
                constexpr uint32_t idesc_s = instr_desc(ROWS, KEYS, 1, 1, 0, 0);
                constexpr uint32_t idesc_o = instr_desc(ROWS, D, 1, 1, 0, 1);   // V is MN-major
                const uint32_t sq = smem_u32(smem + L::Q), sk = smem_u32(smem + L::K);
                const uint32_t sv = smem_u32(smem + L::V);
                auto issue_s = [&](int j) {
                    const int b = j & 1;
                    if (!mbar_wait(k_full, j & 1, ab, 203)) return;
                    // Buffer b still holds P(j-2) as the A operand of P.V(j-2).  Consecutive MMAs overlap in
                    // the tensor pipe, so issue order alone does not protect it: wait for that P.V to finish.
                    if (j >= 2 && !mbar_wait(pv_done, j & 1, ab, 204)) return;
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
                };
                if (mbar_wait(q_full, 0, ab, 205)) {
                    issue_s(0);
                    for (int j = 0; j < n_tiles; ++j) {
                        if (j + 1 < n_tiles) issue_s(j + 1);
                        if (!mbar_wait(p_full, j & 1, ab, 206)) break;
                        if (!mbar_wait(v_full, j & 1, ab, 207)) break;
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < KEYS / 16; ++kk) {
                            uint64_t db = smem_desc_sw128(sv + kk * 2048, SLAB, 1024);
                            mma_bf16_ts(tmem_o, tmem_base + (j & 1) * KEYS + kk * 8, db, idesc_o, (j | kk) != 0);
                        }
                        mma_commit(pv_done);
                        mma_commit(v_empty);
                    }
                }
            }
        } else {
            // ------------------------------------------------------------ softmax + epilogue (warps 2..5)
            const int part = warp & 3;
            const int row = part * 32 + lane;
            const int tok_local = row / G;
            const int head = kvh * G + row % G;
            const bool row_valid = tok_local < q_count;
            const int64_t token = int64_t(q_start) + tok_local;
            const int rlo = row_valid ? p.row_lo[token] : 0;
            const int rhi = row_valid ? p.row_hi[token] : 0;
            const uint32_t lane_addr = uint32_t(part * 32) << 16;
            const float c = p.scale_log2;
            const float lazy = LAZY_LOG2 / c;
            float m_ref = -INFINITY, l = 0.f;

            for (int j = 0; j < n_tiles; ++j) {
                const int b = j & 1;
                if (!mbar_wait(&s_full[b], (j >> 1) & 1, ab, 208)) break;
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
                // P(j) may only be stored once P.V(j-1) has completed: a tcgen05.st into tensor memory while a
                // TS-form MMA is still reading its A operand from tensor memory corrupted results on B200, even
                // though the two touch different columns.  The same wait makes O stable for a rescale.
                if (j > 0) {
                    mbar_wait(pv_done, (j - 1) & 1, ab, 209);
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
                if (lane == 0) mbar_arrive(p_full);
            }

            // epilogue: O / l -> bf16
            if (mbar_wait(pv_done, (n_tiles - 1) & 1, ab, 210)) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16* dst = p.out + (token * p.q_heads + head) * D;
                // a tensor-memory load takes some hundred cycles to return: up to four are in flight per wait
                constexpr int EP = D < 128 ? D : 128;
#pragma unroll 1
                for (int half = 0; half < D; half += EP) {
                    uint32_t o[EP];
#pragma unroll
                    for (int cc = 0; cc < EP; cc += 32) tmem_ld32(tmem_o + lane_addr + half + cc, o + cc);
                    tmem_wait_ld();
                    if (row_valid) {
#pragma unroll
                        for (int v4 = 0; v4 < EP / 8; ++v4) {
                            uint4 v;
                            v.x = pack_bf16(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                            v.y = pack_bf16(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                            v.z = pack_bf16(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                            v.w = pack_bf16(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + half + v4 * 8) = v;
                        }
                    }
                }
                if (p.lse != nullptr && row_valid) {
                    const float ln2 = 0.6931471805599453f;
                    p.lse[int64_t(head) * p.tq + token] =
                        l > 0.f ? (m_ref * c + log2f(l)) * ln2 : -INFINITY;
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
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mck,
           const CUtensorMap& mcv, const AttnParams& p, int n_tiles, cudaStream_t stream) {
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
    dim3 grid((unsigned)n_tiles, (unsigned)p.kv_heads);
    cudaError_t e = launch_kernel(varlen_attention_kernel<D>, grid, dim3(THREADS), Smem<D>::TOTAL, stream, 0, mq, mk, mv,
                                  mck, mcv, p);
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

    AttnParams p;
    p.tiles = tiles; p.row_lo = row_lo; p.row_hi = row_hi;
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse; p.tq = tq;
    p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = bg_status_word();
    if (!p.status) return BG_ERR_DRIVER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return head_dim == 64 ? launch<64>(mq, mk, mv, mck, mcv, p, n_tiles, s)
                          : launch<256>(mq, mk, mv, mck, mcv, p, n_tiles, s);
}
