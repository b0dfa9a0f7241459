// Single-query (decode) attention with grouped queries, split over the KV length.
//
// Work item = (batch row, kv head, KV split); one CTA of four warps each.  The
// CTA streams its keys and values once, 64 keys per tile, through a 3-deep ring
// of shared-memory stages filled with 16-byte cp.async copies (zero-filled past
// the row's valid length, XOR-swizzled so that ldmatrix is conflict free).  The
// G query heads that share the kv head form the rows of a 16-row mma tile
// (rows >= G are zero), so every K/V byte is used by all G heads while it is on
// chip: S = Q K^T and O += P V both run on mma.sync m16n8k16 with fp32
// accumulation, soft-max statistics in fp32 in the exp2 domain.  Each warp owns
// 16 of the tile's 64 keys with its own running (max, sum, O); the four are
// merged in shared memory at the end, the split's (max, sum, O) goes to the
// workspace, and the CTA that finishes last for a (row, kv head) -- found with
// one atomic counter, no waiting -- folds the splits together in index order
// and writes the bf16 output.  No spin waits anywhere.
//
// Decode-layer mode (fuse_new_token): q, k, v of the token being decoded come
// straight from the fused QKV projection output; q and k get their RMSNorm over
// the head here (optionally with a weight and the rotary embedding, fp32 with one
// rounding), and the CTA whose split holds the token's cache slot (S-1, or the
// row's own length - 1 when per-row lengths are given) writes the new k and v
// into the cache and patches them into its shared-memory tile.
// The caches are contiguous [B, NKV, S, D] or page pools addressed through a page
// table (pages of a power-of-two number of keys >= 64, so a tile never straddles
// pages).
#include "launchers.h"

namespace ezb {

static constexpr int kAttnThreads = 128;
static constexpr int kTileKeys = 64;
static constexpr int kAttnStages = 3;

struct AttnParams {
    const bf16* Q;
    long long q_bstride;
    const bf16* K;
    const bf16* V;
    bf16* Out;
    long long o_bstride;
    const int* seq_lens;
    int B, H, NKV, S, G;
    int chunk, nchunks, nqt;
    float scale_log2e;
    float* part_o;   // [items][16][D]
    float* part_ml;  // [items][16][2]
    unsigned int* counters;
    int fuse_new_token;
    const bf16* qkv;
    long long qkv_bstride;
    int q_rows, kv_rows;
    bf16* K_cache_w;
    bf16* V_cache_w;
    float eps;
    const bf16* q_norm_w;
    const bf16* k_norm_w;
    const bf16* rope_cos;
    const bf16* rope_sin;
    int rope_by_len;  // 1: rope_cos / rope_sin are table bases, the row used is the token's slot (len-1)
    const int* page_table;  // null: contiguous caches [B, NKV, S, D]; else [B, max_pages] page ids into pools [pages, NKV, P, D]
    int page_shift;         // log2 of the page size P (a power of two >= 64, so a 64-key tile never straddles pages)
    int max_pages;
    int num_pages;          // pages in the pools: a table entry outside [0, num_pages) is reported, never dereferenced
    unsigned int* status;
    PrefetchList next;
    Trace trace;
};

// Head RMSNorm (+ optional weight, + optional rotate-half RoPE) of one head held by a warp:
// lane owns elements lane + 32*j, so the rotation partner (i +- D/2) is in the same lane.
// x: in/out fp32 values; returns them ready for the single bf16 rounding.
template <int D>
__device__ __forceinline__ void head_norm_rope(float (&x)[D / 32], float eps, const bf16* w, const bf16* cosr, const bf16* sinr,
                                               int lane) {
    constexpr int NJ = D / 32, HJ = NJ / 2;
    float ssq = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) ssq += x[j] * x[j];
    ssq = warp_sum(ssq);
    const float r = 1.0f / sqrtf(ssq / (float)D + eps);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        x[j] = __fmul_rn(x[j], r);
        if (w) x[j] = __fmul_rn(x[j], __bfloat162float(w[lane + j * 32]));
    }
    if (cosr) {
#pragma unroll
        for (int j = 0; j < HJ; ++j) {
            const int i = lane + j * 32, i2 = i + D / 2;
            const float n1 = x[j], n2 = x[j + HJ];
            x[j] = __fadd_rn(__fmul_rn(n1, __bfloat162float(cosr[i])), __fmul_rn(-n2, __bfloat162float(sinr[i])));
            x[j + HJ] = __fadd_rn(__fmul_rn(n2, __bfloat162float(cosr[i2])), __fmul_rn(n1, __bfloat162float(sinr[i2])));
        }
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 2) attn_decode_kernel(const AttnParams p) {
    constexpr int CPR = D / 8;                       // 16-byte chunks per key row
    constexpr int ROW_BYTES = D * 2;
    constexpr int TILE_BYTES = kTileKeys * ROW_BYTES;  // one K or V tile
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int QS = D + 8;                        // padded query row, elements
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stages = smem;
    bf16* q_s = reinterpret_cast<bf16*>(smem + kAttnStages * STAGE_BYTES);
    bf16* kv_new_s = q_s + 16 * QS;  // [2][D]: the new token's k (normalised) and v, decode-layer mode
    __shared__ int s_is_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g4 = lane >> 2, t4 = lane & 3;
    const int chunk_id = blockIdx.x % p.nchunks, qt = blockIdx.x / p.nchunks;
    const int kvh = blockIdx.y, b = blockIdx.z;
    const int G = p.G, g0 = qt * 16, gn = min(16, G - g0);
    const long long kv_row0 = ((long long)b * p.NKV + kvh) * p.S;
    // Row (in units of D elements) of this (batch row, kv head)'s key `key` in the cache.
    // A page id outside the pools (a stale or "unallocated" -1 entry) sets ok = false and records a fault; the
    // caller then touches no memory for that key.
    auto cache_row = [&](int key, bool& ok) -> long long {
        if (!p.page_table) return kv_row0 + key;
        const long long page = __ldg(p.page_table + (long long)b * p.max_pages + (key >> p.page_shift));
        if (page < 0 || page >= p.num_pages) {
            if (ok) report_fault(p.status, FAULT_PAGE_RANGE);
            ok = false;
            return 0;
        }
        return ((page * p.NKV + kvh) << p.page_shift) + (key & ((1 << p.page_shift) - 1));
    };

    unsigned long long* trec = (tid == 0) ? trace_open(p.trace, 9u, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) : nullptr;
    pdl_trigger();
    // This kernel is latency-bound at small batch; meanwhile HBM can already pull
    // the next kernel's weights (immutable, so safe before the dependency wait).
    if (warp == 3) prefetch_next_operands(p.next, lane, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                                         gridDim.x * gridDim.y * gridDim.z);
    // The KV cache is mutable state (an earlier kernel in the stream may have
    // written a slot of it), so nothing is read before the dependency wait.
    pdl_wait();
    trace_mark(trec, 3);

    // The first tiles are requested right away, so that their latency overlaps
    // the query prologue below.
    int len = p.S;
    if (p.seq_lens) len = max(p.fuse_new_token ? 1 : 0, min(p.S, p.seq_lens[b]));
    // decode-layer mode: the token being decoded is the last valid key of the row (slot len-1;
    // with one length for all rows that is slot S-1, the reference layer's convention)
    const int new_slot = len - 1;
    const bf16* rope_cos = p.rope_cos ? p.rope_cos + (p.rope_by_len ? (long long)new_slot * D : 0) : nullptr;
    const bf16* rope_sin = p.rope_sin ? p.rope_sin + (p.rope_by_len ? (long long)new_slot * D : 0) : nullptr;
    const int c0 = chunk_id * p.chunk;
    const int c1 = min(len, c0 + p.chunk);
    const int nkeys = max(0, c1 - c0);
    const int ntiles = (nkeys + kTileKeys - 1) / kTileKeys;
    const bool owns_new_slot = p.fuse_new_token && c0 <= new_slot && new_slot < c1;

    auto load_tile = [&](int t) {
        unsigned char* st = stages + (t % kAttnStages) * STAGE_BYTES;
        const int key0 = c0 + t * kTileKeys;
        bool page_ok = true;
        const long long tile_row0 = cache_row(key0, page_ok);  // the tile lies inside one page
#pragma unroll
        for (int i = 0; i < (2 * kTileKeys * CPR) / kAttnThreads; ++i) {
            const int idx = tid + i * kAttnThreads;
            const int which = idx / (kTileKeys * CPR);
            const int rem = idx % (kTileKeys * CPR);
            const int r = rem / CPR, c = rem % CPR;
            const int key = key0 + r;
            const bool valid = page_ok && key < c1;  // a tile of a bad page is zero-filled, nothing is read
            const bf16* src = (which ? p.V : p.K) + (tile_row0 + (valid ? r : 0)) * D + c * 8;
            const uint32_t dst = smem_u32(st) + which * TILE_BYTES + r * ROW_BYTES + ((c ^ (r & 7)) << 4);
            cp_async16(dst, src, valid);
        }
    };
    // Tiles of the start-up window (one commit group per tile, in tile order).
    // In decode-layer mode slot S-1 still holds stale data when its tile is
    // requested; the CTA that owns it overwrites that row in shared memory once
    // the tile has landed (see the loop below), so it needs no global round trip.
    const int early = min(kAttnStages - 1, ntiles);
    for (int t = 0; t < early; ++t) {
        load_tile(t);
        cp_async_commit();
    }

    // ---- queries of this kv group into shared memory (rows >= gn are zero) ----
    {
        const bf16* qsrc = p.fuse_new_token ? p.qkv : p.Q;
        const long long qb = p.fuse_new_token ? p.qkv_bstride : p.q_bstride;
        constexpr int QV = (16 * CPR + kAttnThreads - 1) / kAttnThreads;
        uint4 qv[QV];
#pragma unroll
        for (int u = 0; u < QV; ++u) {  // loads first, stores after: one L2 round trip
            const int idx = tid + u * kAttnThreads;
            const int row = idx / CPR, c = idx % CPR;
            qv[u] = make_uint4(0, 0, 0, 0);
            if (idx < 16 * CPR && row < gn)
                qv[u] = *reinterpret_cast<const uint4*>(qsrc + (long long)b * qb + (long long)(kvh * G + g0 + row) * D + c * 8);
        }
#pragma unroll
        for (int u = 0; u < QV; ++u) {
            const int idx = tid + u * kAttnThreads;
            if (idx < 16 * CPR) *reinterpret_cast<uint4*>(q_s + (idx / CPR) * QS + (idx % CPR) * 8) = qv[u];
        }
        __syncthreads();
        if (p.fuse_new_token) {
            // unit-weight RMSNorm over the head, fp32 statistics, one rounding
            for (int row = warp; row < gn; row += 4) {
                float x[D / 32];
#pragma unroll
                for (int j = 0; j < D / 32; ++j) x[j] = __bfloat162float(q_s[row * QS + lane + j * 32]);
                head_norm_rope<D>(x, p.eps, p.q_norm_w, rope_cos, rope_sin, lane);
#pragma unroll
                for (int j = 0; j < D / 32; ++j) q_s[row * QS + lane + j * 32] = __float2bfloat16_rn(x[j]);
            }
            // new token's k (normalised) and v: kept in shared memory for the patch below and
            // written to cache slot S-1 (nobody reads that slot from memory in this kernel)
            if (owns_new_slot) {
                bool slot_ok = true;
                const long long slot = cache_row(new_slot, slot_ok) * D;
                const bool write_slot = slot_ok && qt == 0;  // a bad page: the new k / v are not written anywhere
                if (warp == 0) {
                    const bf16* ksrc = p.qkv + (long long)b * p.qkv_bstride + p.q_rows + kvh * D;
                    float x[D / 32];
#pragma unroll
                    for (int j = 0; j < D / 32; ++j) x[j] = __bfloat162float(ksrc[lane + j * 32]);
                    head_norm_rope<D>(x, p.eps, p.k_norm_w, rope_cos, rope_sin, lane);
#pragma unroll
                    for (int j = 0; j < D / 32; ++j) {
                        const bf16 kn = __float2bfloat16_rn(x[j]);
                        kv_new_s[lane + j * 32] = kn;
                        if (write_slot) p.K_cache_w[slot + lane + j * 32] = kn;
                    }
                } else if (warp == 1) {
                    const bf16* vsrc = p.qkv + (long long)b * p.qkv_bstride + p.q_rows + p.kv_rows + kvh * D;
#pragma unroll
                    for (int j = 0; j < D / 32; ++j) {
                        const bf16 vn = vsrc[lane + j * 32];
                        kv_new_s[D + lane + j * 32] = vn;
                        if (write_slot) p.V_cache_w[slot + lane + j * 32] = vn;
                    }
                }
            }
            __syncthreads();
        }
    }

    // ---- A fragments of Q: 16 rows x D, D/16 k-steps ----
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        const bf16* base = q_s + kk * 16 + t4 * 2;
        qa[kk][0] = *reinterpret_cast<const uint32_t*>(base + g4 * QS);
        qa[kk][1] = *reinterpret_cast<const uint32_t*>(base + (g4 + 8) * QS);
        qa[kk][2] = *reinterpret_cast<const uint32_t*>(base + g4 * QS + 8);
        qa[kk][3] = *reinterpret_cast<const uint32_t*>(base + (g4 + 8) * QS + 8);
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};

    for (int t = early; t < kAttnStages - 1; ++t) {
        if (t < ntiles) load_tile(t);
        cp_async_commit();
    }
    for (int t = 0; t < ntiles; ++t) {
        cp_async_wait<kAttnStages - 2>();
        __syncthreads();
        if (t == 0) trace_mark(trec, 4);
        if (t + kAttnStages - 1 < ntiles) load_tile(t + kAttnStages - 1);
        cp_async_commit();
        if (owns_new_slot && t == ntiles - 1) {
            // overwrite the stale row of slot S-1 in this tile with the new token's k and v
            const int r = new_slot - (c0 + t * kTileKeys);
            if (tid < 2 * CPR) {
                const int which = tid / CPR, c = tid % CPR;
                unsigned char* dst = stages + (t % kAttnStages) * STAGE_BYTES + which * TILE_BYTES + r * ROW_BYTES + ((c ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(kv_new_s + which * D + c * 8);
            }
            __syncthreads();
        }

        const unsigned char* st = stages + (t % kAttnStages) * STAGE_BYTES;
        const uint32_t k_s = smem_u32(st), v_s = k_s + TILE_BYTES;
        const int kr0 = warp * 16;

        // ---- S = Q K^T for this warp's 16 keys ----
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const int mi = lane >> 3, rr = lane & 7;
            const int key_local = kr0 + (mi >> 1) * 8 + rr;
            const uint32_t row_addr = k_s + key_local * ROW_BYTES;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int chunk = kk * 2 + (mi & 1);
                uint32_t b00, b01, b10, b11;
                ldsm_x4(row_addr + ((chunk ^ (key_local & 7)) << 4), b00, b01, b10, b11);
                mma_bf16_16816(s[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b00, b01);
                mma_bf16_16816(s[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b10, b11);
            }
        }
        // ---- online soft-max (exp2 domain) ----
        const int key_base = c0 + t * kTileKeys + kr0 + t4 * 2;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key_base + j * 8 + (e & 1);
                s[j][e] = (key < c1) ? s[j][e] * p.scale_log2e : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
            }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[r] = fast_exp2(m_run[r] - m_safe);
            m_run[r] = m_new;
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][2 * r] = fast_exp2(s[j][2 * r] - m_safe);
                s[j][2 * r + 1] = fast_exp2(s[j][2 * r + 1] - m_safe);
                psum += s[j][2 * r] + s[j][2 * r + 1];
            }
            l_run[r] = l_run[r] * alpha[r] + psum;
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= alpha[0], o[i][1] *= alpha[0];
            o[i][2] *= alpha[1], o[i][3] *= alpha[1];
        }
        // ---- O += P V ----
        const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]), pa1 = pack_bf16(s[0][2], s[0][3]);
        const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]), pa3 = pack_bf16(s[1][2], s[1][3]);
        {
            const int mi = lane >> 3, rr = lane & 7;
            const int key_local = kr0 + (mi & 1) * 8 + rr;
            const uint32_t row_addr = v_s + key_local * ROW_BYTES;
#pragma unroll
            for (int dn = 0; dn < D / 16; ++dn) {
                const int chunk = dn * 2 + (mi >> 1);
                uint32_t v0, v1, v2, v3;
                ldsm_x4_trans(row_addr + ((chunk ^ (key_local & 7)) << 4), v0, v1, v2, v3);
                mma_bf16_16816(o[2 * dn], pa0, pa1, pa2, pa3, v0, v1);
                mma_bf16_16816(o[2 * dn + 1], pa0, pa1, pa2, pa3, v2, v3);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the four warps (each saw a quarter of the keys) ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* mrg_m = reinterpret_cast<float*>(smem);  // [4][16]
    float* mrg_l = mrg_m + 64;                      // [4][16]
    float* mrg_o = mrg_l + 64;                      // [4][16][D]
    if (t4 == 0) {
        mrg_m[warp * 16 + g4] = m_run[0], mrg_m[warp * 16 + g4 + 8] = m_run[1];
        mrg_l[warp * 16 + g4] = l_run[0], mrg_l[warp * 16 + g4 + 8] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        float* dst = mrg_o + (warp * 16 + g4) * D + i * 8 + t4 * 2;
        *reinterpret_cast<float2*>(dst) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(dst + 8 * D) = make_float2(o[i][2], o[i][3]);
    }
    __syncthreads();

    const long long group = ((long long)b * p.NKV + kvh) * p.nqt + qt;
    const long long item = group * p.nchunks + chunk_id;
    for (int idx = tid; idx < gn * D; idx += kAttnThreads) {
        const int row = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mrg_m[w * 16 + row]);
        float O = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = fast_exp2(mrg_m[w * 16 + row] - M);
                O += f * mrg_o[(w * 16 + row) * D + d];
                L += f * mrg_l[w * 16 + row];
            }
        }
        if (p.nchunks == 1) {
            const float val = (L > 0.f) ? O / L : 0.f;
            p.Out[(long long)b * p.o_bstride + (long long)(kvh * G + g0 + row) * D + d] = __float2bfloat16_rn(val);
        } else {
            p.part_o[(item * 16 + row) * D + d] = O;
            if (d == 0) {
                p.part_ml[(item * 16 + row) * 2 + 0] = M;
                p.part_ml[(item * 16 + row) * 2 + 1] = L;
            }
        }
    }
    if (p.nchunks == 1) {
        trace_mark(trec, 5);
        return;
    }

    // ---- the last CTA of this (row, kv head, q tile) folds the splits together ----
    // One acq_rel atomic after the barrier both publishes this CTA's records (the
    // barrier orders the other threads' stores before it) and, for the CTA that
    // draws the last ticket, makes every other CTA's records visible.
    __syncthreads();
    if (tid == 0) {
        unsigned int prev;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + group) : "memory");
        s_is_last = (prev == (unsigned int)(p.nchunks - 1));
    }
    __syncthreads();
    if (!s_is_last) {
        trace_mark(trec, 5);
        return;
    }
    if (p.nchunks <= 32) {
        // Fast path: every thread owns four output dims of one head and issues all
        // its loads up front (32 split records + the first 16 partial vectors), so
        // the whole fold costs two L2 round trips.
        for (int idx = tid; idx < gn * (D / 4); idx += kAttnThreads) {
            const int row = idx / (D / 4), d = (idx % (D / 4)) * 4;
            const float* pm = p.part_ml + ((group * p.nchunks) * 16 + row) * 2;
            const float* po = p.part_o + ((group * p.nchunks) * 16 + row) * D + d;
            float2 ml[32];
            float4 v[16];
#pragma unroll
            for (int c = 0; c < 32; ++c)
                ml[c] = (c < p.nchunks) ? __ldcg(reinterpret_cast<const float2*>(pm + (long long)c * 32)) : make_float2(-INFINITY, 0.f);
#pragma unroll
            for (int c = 0; c < 16; ++c)
                v[c] = (c < p.nchunks) ? __ldcg(reinterpret_cast<const float4*>(po + (long long)c * 16 * D)) : make_float4(0.f, 0.f, 0.f, 0.f);
            float M = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c) M = fmaxf(M, ml[c].x);
            float L = 0.f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                ml[c].x = (M != -INFINITY) ? fast_exp2(ml[c].x - M) : 0.f;
                L += ml[c].x * ml[c].y;
            }
            const float inv = (L > 0.f) ? 1.0f / L : 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float f = ml[c].x;
                acc.x += f * v[c].x, acc.y += f * v[c].y, acc.z += f * v[c].z, acc.w += f * v[c].w;
            }
            if (p.nchunks > 16) {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    v[c] = (c + 16 < p.nchunks) ? __ldcg(reinterpret_cast<const float4*>(po + (long long)(c + 16) * 16 * D))
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float f = ml[c + 16].x;
                    acc.x += f * v[c].x, acc.y += f * v[c].y, acc.z += f * v[c].z, acc.w += f * v[c].w;
                }
            }
            bf16* dst = p.Out + (long long)b * p.o_bstride + (long long)(kvh * G + g0 + row) * D + d;
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
    } else {
        // General path: split weights through shared memory.
        float* cm = reinterpret_cast<float*>(smem);        // [nchunks][16] split maxima, then weights
        float* cl = cm + (size_t)p.nchunks * 16;           // [nchunks][16] split sums
        for (int idx = tid; idx < p.nchunks * gn; idx += kAttnThreads) {
            const int c = idx / gn, row = idx % gn;
            const long long rec = ((group * p.nchunks + c) * 16 + row) * 2;
            cm[c * 16 + row] = __ldcg(&p.part_ml[rec]);
            cl[c * 16 + row] = __ldcg(&p.part_ml[rec + 1]);
        }
        __syncthreads();
        for (int row = warp; row < gn; row += 4) {  // one warp per head, lanes over splits
            float M = -INFINITY;
            for (int c = lane; c < p.nchunks; c += 32) M = fmaxf(M, cm[c * 16 + row]);
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
            float L = 0.f;
            if (M != -INFINITY)
                for (int c = lane; c < p.nchunks; c += 32) L += fast_exp2(cm[c * 16 + row] - M) * cl[c * 16 + row];
            L = warp_sum(L);
            const float inv = (L > 0.f) ? 1.0f / L : 0.f;
            for (int c = lane; c < p.nchunks; c += 32)
                cm[c * 16 + row] = (M != -INFINITY) ? fast_exp2(cm[c * 16 + row] - M) * inv : 0.f;
        }
        __syncthreads();
        for (int idx = tid; idx < gn * (D / 4); idx += kAttnThreads) {
            const int row = idx / (D / 4), d = (idx % (D / 4)) * 4;
            const float* po = p.part_o + ((group * p.nchunks) * 16 + row) * D + d;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = 0; c < p.nchunks; c += 16) {
                float4 v[16];
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    v[u] = (c + u < p.nchunks) ? __ldcg(reinterpret_cast<const float4*>(po + (long long)(c + u) * 16 * D))
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const float f = (c + u < p.nchunks) ? cm[(c + u) * 16 + row] : 0.f;
                    acc.x += f * v[u].x, acc.y += f * v[u].y, acc.z += f * v[u].z, acc.w += f * v[u].w;
                }
            }
            bf16* dst = p.Out + (long long)b * p.o_bstride + (long long)(kvh * G + g0 + row) * D + d;
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
        }
    }
    if (tid == 0) p.counters[group] = 0u;  // ready for the next call
    trace_mark(trec, 5);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// Rows of equal length are cut so that all CTAs are resident together, in ONE wave: as many splits per (row, kv
// head) as the resident slots allow, never more.  A second, partly filled wave costs a whole extra pass over a split
// (Qwen3-8B layer, KV 4096, batch 2 / 4 / 8 / 16 / 32: 94.5 / 110.5 / 126.8 / 147.1 / 191.4 us with splits sized for
// 1.5 waves, 89.5 / 107.4 / 124.6 / 141.2 / 181.6 with this rule; a sweep over every split length confirmed the
// optimum at ~256 CTAs for each).  Ragged batches are cut into more, shorter splits, because every row is cut on
// the grid of the longest row and short splits balance better.
int attn_chunk_keys(int B, int NKV, int S, bool ragged, int D) {
    const long long total = (long long)B * NKV * S;
    const int waves = tuning(ragged ? EZB_TUNE_ATTN_WAVES : EZB_TUNE_ATTN_WAVES_UNIFORM);
    long long chunk;
    if (!ragged && waves <= 0) {
        const long long slots = (long long)sm_count() * (D <= 64 ? 4 : 2);  // resident CTAs: the ring is 3 x 2 x 64 keys x D
        long long splits = slots / ((long long)B * NKV);
        if (splits < 1) splits = 1;
        chunk = (S + splits - 1) / splits;
    } else {
        const long long target = (long long)sm_count() * max(1, waves);
        chunk = (total + target - 1) / target;
    }
    chunk = (chunk + kTileKeys - 1) / kTileKeys * kTileKeys;
    long long floor_keys = max(kTileKeys, tuning(EZB_TUNE_ATTN_MIN_CHUNK) / kTileKeys * kTileKeys);
    if (chunk < floor_keys) chunk = floor_keys;
    const long long cap = ((long long)S + kTileKeys - 1) / kTileKeys * kTileKeys;
    if (chunk > cap) chunk = cap;
    // the combine keeps two floats per (split, head) in shared memory
    while ((S + chunk - 1) / chunk > 256) chunk += kTileKeys;
    return (int)chunk;
}

static size_t counters_bytes(int B, int NKV, int nqt) { return ((size_t)B * NKV * nqt * 4 + 255) / 256 * 256; }

size_t attn_counters_bytes(int B, int H, int NKV) {
    const int G = H / NKV;
    return counters_bytes(B, NKV, (G + 15) / 16);
}

size_t attn_workspace_bytes(int B, int H, int NKV, int S, int D) {
    const int G = H / NKV, nqt = (G + 15) / 16;
    const int chunk = min(attn_chunk_keys(B, NKV, S, false, D), attn_chunk_keys(B, NKV, S, true, D));  // covers both cuts
    const int nchunks = (S + chunk - 1) / chunk;
    const size_t items = (size_t)B * NKV * nqt * nchunks;
    return counters_bytes(B, NKV, nqt) + items * 16 * 2 * sizeof(float) + items * 16 * D * sizeof(float);
}

template <int D>
static cudaError_t launch_attn_instance(const AttnParams& p, cudaStream_t stream) {
    auto kernel = attn_decode_kernel<D>;
    constexpr size_t smem = (size_t)kAttnStages * 2 * kTileKeys * D * 2 + 16 * (D + 8) * 2 + 2 * D * 2;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(p.nchunks * p.nqt, p.NKV, p.B), dim3(kAttnThreads), smem, stream, p);
}

cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream) {
    AttnParams p;
    p.Q = a.Q, p.q_bstride = a.q_bstride, p.K = a.K, p.V = a.V, p.Out = a.Out, p.o_bstride = a.o_bstride;
    p.seq_lens = a.seq_lens;
    p.B = a.B, p.H = a.H, p.NKV = a.NKV, p.S = a.S, p.G = a.H / a.NKV;
    p.nqt = (p.G + 15) / 16;
    p.chunk = attn_chunk_keys(a.B, a.NKV, a.S, a.seq_lens != nullptr, a.D);
    p.nchunks = (a.S + p.chunk - 1) / p.chunk;
    p.scale_log2e = 1.4426950408889634f / sqrtf((float)a.D);
    unsigned char* ws = reinterpret_cast<unsigned char*>(a.workspace);
    const size_t items = (size_t)a.B * a.NKV * p.nqt * p.nchunks;
    p.counters = reinterpret_cast<unsigned int*>(ws);
    p.part_ml = reinterpret_cast<float*>(ws + counters_bytes(a.B, a.NKV, p.nqt));
    p.part_o = p.part_ml + items * 16 * 2;
    p.fuse_new_token = a.fuse_new_token;
    p.qkv = a.qkv, p.qkv_bstride = a.qkv_bstride;
    p.q_rows = a.H * a.D, p.kv_rows = a.NKV * a.D;
    p.K_cache_w = a.K_cache_w, p.V_cache_w = a.V_cache_w;
    p.eps = a.eps;
    p.q_norm_w = a.q_norm_w, p.k_norm_w = a.k_norm_w, p.rope_cos = a.rope_cos, p.rope_sin = a.rope_sin;
    p.rope_by_len = a.rope_by_len;
    p.page_table = a.page_table, p.page_shift = a.page_shift, p.max_pages = a.max_pages, p.num_pages = a.num_pages;
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    p.next = a.next;
    if (!tuning(EZB_TUNE_L2_PREFETCH)) p.next.plan[0].units = p.next.plan[1].units = 0;
    p.trace = trace_handle();
    if (a.D == 128) return launch_attn_instance<128>(p, stream);
    return launch_attn_instance<64>(p, stream);
}

}  // namespace ezb
