// Windowed attention over the paged cache on the tensor cores (bfloat16 operands, float32
// scores, weights and sums), for mixers whose sizes are parameters: keys TILES_KEY_DIM wide,
// values TILES_VALUE_DIM wide (both multiples of 16; the library is compiled per pair), a
// sliding window that may keep the first `keep_first` keys visible, an optional output gate (one number
// a value, or one a head), an optional distance bias (head h takes slopes[h] * (p - j) off the score of
// key j) and an optional sink a head (exp(sink) is added to the softmax's denominator and to nothing
// else), an optional learned bias by distance (bias_table[min(p - j, rows - 1), h] is added to the scaled
// score) and optional segments (a query sees only the keys from the start of its own segment of
// `segment` positions, counted from position 0; not together with a window).  Compiled with TILES_VALUE_IN_KEY=1 the values are the first TILES_VALUE_DIM elements of the
// key rows themselves (attention over latents that serve as keys and values): no value cache is read
// and the key tile in shared memory is the value tile too.
//
// The query at position p sees key j iff j <= p and (window == 0 or p - j < window or
// j < keep_first).  A CTA of 4 warps holds up to 64 query rows (16 a warp) that share one
// request and one kv head, walks the keys they see in tiles of 32 that start at absolute
// multiples of 32 (first the tiles of kept first keys that lie before the window, then the
// window's), K and V tiles coming in through two cp.async stages, S = Q K^T and O += P V on
// mma.sync m16n8k16.  The weights P stay float32: each is cut into a bfloat16 head and a
// bfloat16 rest (p = hi + lo, exact to 2^-17 of p) and both halves are multiplied with V, so
// nothing of a weight is lost before the float32 sum; the denominator sums the float32 values.
//
// Two forms of a CTA's rows:
//   tiles    rows = up to 64 consecutive tokens of one prompt portion, one q head (grid: tiles
//            x q heads); the result is divided, gated and stored.
//   singles  rows = the q heads of one kv head for ONE token (decoded tokens; up to 64 heads a
//            group); the token's keys are cut into chunks of 128 at absolute multiples of 128,
//            a CTA takes one chunk (grid: tokens x kv heads x chunks, chunks counted back from
//            the token's own position, then the chunks of kept first keys) and leaves
//            (max, sum, out) in scratch; a second kernel merges a row's chunks in ascending
//            order, gates and stores.  The keys are read once per kv head, and what a row sums
//            depends on its own position only, not on the batch it is in.  With up to 16 heads a
//            group the chunk comes in with one wave of copies and every warp takes 32 of its
//            keys (attention_singles_kernel); larger groups walk the chunk tile by tile.
#include "common.cuh"

#ifndef TILES_KEY_DIM
#define TILES_KEY_DIM 64
#endif
#ifndef TILES_VALUE_DIM
#define TILES_VALUE_DIM 64
#endif

#ifndef TILES_VALUE_IN_KEY
#define TILES_VALUE_IN_KEY 0
#endif

#define TL_BM 64
#define TL_BN 32
#define TL_WARPS 4
#define TL_PAD 8
#define TL_CHUNK 128           // keys per CTA in the singles form
#define TL_LOG2E 1.4426950408889634f

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// p = hi + lo with hi = bf16(p), lo = bf16(p - hi)
__device__ __forceinline__ void split_pair(float p0, float p1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
    const float2 back = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(p0 - back.x, p1 - back.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ float sigmoid_of(float g) { return __fdiv_rn(1.0f, 1.0f + expf(-g)); }

struct TileArgs {
    const bf16* q; long long q_token_stride;
    const bf16* key_cache; const bf16* value_cache;
    const int* block_tables; int table_stride;
    const int* positions; const int* token_row;
    const int* tile_row; const int* tile_first; const int* tile_count;
    bf16* out; long long out_token_stride;
    const bf16* gate; long long gate_token_stride;
    float* scratch; int window_chunks; int kept_chunks;
    int num_q, num_kv, page_size, window, keep_first;
    float scale;
    const float* slopes; const float* sinks; int gate_per_head;
    const float* bias_table; int bias_rows; int segment;
};

// The first key the query at `position` sees (kept first keys apart): the start of its segment of
// `segment` positions counted from 0, or the far end of its window, or 0.
__device__ __forceinline__ int lowest_seen(const TileArgs& a, int position) {
    if (a.segment > 0) return position - position % a.segment;
    return a.window > 0 ? max(0, position - a.window + 1) : 0;
}

// table[min(distance, rows - 1), head] in the units of the scaled scores
__device__ __forceinline__ float table_bias(const TileArgs& a, int distance, int head) {
    return __ldg(a.bias_table + (int64_t)min(max(distance, 0), a.bias_rows - 1) * a.num_q + head) * TL_LOG2E;
}

__device__ __forceinline__ int chunk_of_slot(int z, int window_chunks, int position, int lo, int kept);

template <int KD, int VD, bool SINGLES>
__global__ void __launch_bounds__(TL_WARPS * 32, 3) attention_tiles_kernel(const TileArgs a) {
    constexpr bool VIK = TILES_VALUE_IN_KEY != 0;
    constexpr int KROW = KD + TL_PAD, VROW = VIK ? KROW : VD + TL_PAD;
    constexpr int KCHUNKS = KD / 8, VCHUNKS = VD / 8;
    extern __shared__ __align__(16) unsigned char shared_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(shared_raw);                         // [64][KROW]
    bf16* k_s = q_s + TL_BM * KROW;                                          // [2][32][KROW]
    bf16* v_s = VIK ? k_s : k_s + 2 * TL_BN * KROW;                          // [2][32][VROW], or the key tiles
    int* slot_s = reinterpret_cast<int*>(VIK ? k_s + 2 * TL_BN * KROW : v_s + 2 * TL_BN * VROW);   // [2][32]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = a.num_q / a.num_kv;
    int request, first_token, count, first_position, kv_head, head0;
    if (SINGLES) {
        first_token = blockIdx.x;
        request = a.token_row[first_token];
        first_position = a.positions[first_token];
        if (request < 0 || first_position < 0) return;        // a padding row; the merge writes its zeros
        kv_head = blockIdx.y;
        head0 = kv_head * group;
        count = group;
    } else {
        const int tile = gridDim.x - 1 - blockIdx.x;         // later tiles see more keys: they start first
        request = a.tile_row[tile], first_token = a.tile_first[tile], count = a.tile_count[tile];
        first_position = a.positions[first_token];
        head0 = blockIdx.y;
        kv_head = head0 / group;
    }
    const int last_position = SINGLES ? first_position : first_position + count - 1;
    const int* table = a.block_tables + (int64_t)request * a.table_stride;
    const bool limited = a.window > 0 || a.segment > 0;
    const int lo_first = lowest_seen(a, first_position);
    const int lo_last = lowest_seen(a, last_position);
    const int kept = min(a.keep_first, lo_last);          // keys 0..kept-1 are seen from behind a window

    // ---- the key tiles this CTA walks: range A (kept first keys before the window), then range B
    int a0 = 0, na = 0, b0, nb;
    {
        const int win_first = lo_first / TL_BN, win_last = last_position / TL_BN;
        const int kept_tiles = min((kept + TL_BN - 1) / TL_BN, win_first);
        if (SINGLES) {
            // chunk of this CTA: z < window_chunks counts back from the token's own chunk; the others are
            // the chunks of kept keys that lie wholly before the window's first chunk
            const int chunk = chunk_of_slot(blockIdx.z, a.window_chunks, first_position, lo_first, kept);
            if (chunk < 0) return;
            const int t0 = chunk * (TL_CHUNK / TL_BN), t1 = t0 + TL_CHUNK / TL_BN - 1;
            na = max(0, min(kept_tiles - 1, t1) - t0 + 1);
            a0 = t0;
            b0 = max(win_first, t0);
            nb = max(0, min(win_last, t1) - b0 + 1);
        } else {
            na = kept_tiles;
            b0 = win_first;
            nb = win_last - win_first + 1;
        }
    }
    const int tiles = na + nb;
    auto key_of_tile = [&](int t) { return (t < na ? a0 + t : b0 + (t - na)) * TL_BN; };

    // ---- Q rows (rows past `count` are zero)
    for (int index = tid; index < TL_BM * KCHUNKS; index += TL_WARPS * 32) {
        const int r = index / KCHUNKS, c = index % KCHUNKS;
        const int rr = min(r, count - 1);
        const bf16* src = SINGLES
            ? a.q + (int64_t)first_token * a.q_token_stride + (int64_t)(head0 + rr) * KD + c * 8
            : a.q + (int64_t)(first_token + rr) * a.q_token_stride + (int64_t)head0 * KD + c * 8;
        cp_async_16(q_s + r * KROW + c * 8, src, r < count);
    }
    cp_async_commit();

    auto stage_slots = [&](int t, int buffer) {
        if (tid < TL_BN) {
            const int key = key_of_tile(t) + tid;
            int slot = -1;
            if (key <= last_position) {
                const int page = table[key / a.page_size];
                if (page >= 0) slot = (page * a.num_kv + kv_head) * a.page_size + key % a.page_size;
            }
            slot_s[buffer * TL_BN + tid] = slot;
        }
    };
    auto load_tile = [&](int buffer) {
        for (int index = tid; index < TL_BN * KCHUNKS; index += TL_WARPS * 32) {
            const int r = index / KCHUNKS, c = index % KCHUNKS;
            const int slot = slot_s[buffer * TL_BN + r];
            cp_async_16(k_s + (buffer * TL_BN + r) * KROW + c * 8,
                        a.key_cache + (int64_t)max(slot, 0) * KD + c * 8, slot >= 0);
        }
        if (!VIK) {
            for (int index = tid; index < TL_BN * VCHUNKS; index += TL_WARPS * 32) {
                const int r = index / VCHUNKS, c = index % VCHUNKS;
                const int slot = slot_s[buffer * TL_BN + r];
                cp_async_16(v_s + (buffer * TL_BN + r) * VROW + c * 8,
                            a.value_cache + (int64_t)max(slot, 0) * VD + c * 8, slot >= 0);
            }
        }
        cp_async_commit();
    };

    if (tiles > 0) stage_slots(0, 0);
    __syncthreads();
    if (tiles > 0) load_tile(0); else cp_async_commit();

    cp_async_wait<1>();                                   // the Q rows (the first group) have landed
    __syncthreads();
    const bool busy = warp * 16 < count;                  // a warp without rows only helps to load
    // this lane's address in the Q rows for ldmatrix: the fragments are read again for every key tile
    // (shared memory has the bandwidth; the registers they would hold let a third CTA onto the SM)
    const bf16* q_lane = q_s + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KROW + (lane >> 4) * 8;

    const int g = lane >> 2, t4 = lane & 3;
    const int row_a = warp * 16 + g, row_b = row_a + 8;
    const int pos_a = SINGLES ? first_position : first_position + row_a;
    const int pos_b = SINGLES ? first_position : first_position + row_b;
    const int lo_a = lowest_seen(a, pos_a);
    const int lo_b = lowest_seen(a, pos_b);
    const int warp_pos_first = SINGLES ? first_position : first_position + warp * 16;
    const int warp_pos_last = SINGLES ? first_position : warp_pos_first + 15;
    float o_acc[VD / 8][4];
#pragma unroll
    for (int n = 0; n < VD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    const float scale_log2 = a.scale * TL_LOG2E;
    // the distance bias of this thread's two rows, in the units of the scaled scores
    const bool biased = a.slopes != nullptr;
    const int head_a = SINGLES ? head0 + min(row_a, count - 1) : head0;
    const int head_b = SINGLES ? head0 + min(row_b, count - 1) : head0;
    const float slope_a = biased ? a.slopes[head_a] * TL_LOG2E : 0.0f;
    const float slope_b = biased ? a.slopes[head_b] * TL_LOG2E : 0.0f;
    const bool tabled = a.bias_table != nullptr;

    for (int t = 0; t < tiles; ++t) {
        const int buffer = t & 1;
        if (t + 1 < tiles) stage_slots(t + 1, buffer ^ 1);
        cp_async_wait<0>();
        __syncthreads();
        if (t + 1 < tiles) load_tile(buffer ^ 1);
        const int key0 = key_of_tile(t);
        // nothing of this tile for this warp's rows: past their diagonal, or before their windows and not kept
        const bool none = key0 > warp_pos_last ||
                          (limited && key0 + TL_BN - 1 < lowest_seen(a, warp_pos_first) && key0 >= a.keep_first);
        if (!busy || none) continue;

        const bf16* k_tile = k_s + buffer * TL_BN * KROW;
        const bf16* v_tile = v_s + buffer * TL_BN * VROW;
        float s_acc[TL_BN / 8][4];
#pragma unroll
        for (int n = 0; n < TL_BN / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KD / 16; ++ks) {
            uint32_t q_frag[4];
            ldmatrix_x4(q_frag, q_lane + ks * 16);
#pragma unroll
            for (int np = 0; np < TL_BN / 16; ++np) {
                uint32_t b[4];
                const int matrix = lane >> 3;
                const int key = np * 16 + (matrix >> 1) * 8 + (lane & 7);
                const int dim = ks * 16 + (matrix & 1) * 8;
                ldmatrix_x4(b, k_tile + key * KROW + dim);
                mma_bf16(s_acc[2 * np], q_frag, b[0], b[1]);
                mma_bf16(s_acc[2 * np + 1], q_frag, b[2], b[3]);
            }
        }

        // every row of the warp sees every key of the tile: below all diagonals and inside all windows
        const bool full = key0 + TL_BN - 1 <= warp_pos_first &&
                          (!limited || key0 >= lowest_seen(a, warp_pos_last));
        float tile_max_a = -INFINITY, tile_max_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < TL_BN / 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = key0 + n * 8 + 2 * t4 + (i & 1);
                const bool upper = i < 2;
                float s = s_acc[n][i] * scale_log2;
                if (biased) s -= (upper ? slope_a : slope_b) * (float)((upper ? pos_a : pos_b) - key);
                if (tabled) s += table_bias(a, (upper ? pos_a : pos_b) - key, upper ? head_a : head_b);
                if (!full) {
                    const int pos = upper ? pos_a : pos_b, lo = upper ? lo_a : lo_b;
                    if (!(key <= pos && (key >= lo || key < a.keep_first))) s = -INFINITY;
                }
                s_acc[n][i] = s;
                if (upper) tile_max_a = fmaxf(tile_max_a, s); else tile_max_b = fmaxf(tile_max_b, s);
            }
        }
        tile_max_a = fmaxf(tile_max_a, __shfl_xor_sync(0xffffffffu, tile_max_a, 1));
        tile_max_a = fmaxf(tile_max_a, __shfl_xor_sync(0xffffffffu, tile_max_a, 2));
        tile_max_b = fmaxf(tile_max_b, __shfl_xor_sync(0xffffffffu, tile_max_b, 1));
        tile_max_b = fmaxf(tile_max_b, __shfl_xor_sync(0xffffffffu, tile_max_b, 2));
        const float new_a = fmaxf(m_a, tile_max_a), new_b = fmaxf(m_b, tile_max_b);
        // a row that has seen no key yet keeps the reference 0 so that no inf - inf appears
        const float ref_a = new_a == -INFINITY ? 0.0f : new_a, ref_b = new_b == -INFINITY ? 0.0f : new_b;
        const float rescale_a = exp2f(m_a - ref_a), rescale_b = exp2f(m_b - ref_b);
        m_a = new_a;
        m_b = new_b;
        float sum_a = 0.0f, sum_b = 0.0f;
        uint32_t p_hi[TL_BN / 16][4], p_lo[TL_BN / 16][4];
#pragma unroll
        for (int n = 0; n < TL_BN / 8; ++n) {
            const float p0 = exp2f(s_acc[n][0] - ref_a), p1 = exp2f(s_acc[n][1] - ref_a);
            const float p2 = exp2f(s_acc[n][2] - ref_b), p3 = exp2f(s_acc[n][3] - ref_b);
            sum_a += p0 + p1;
            sum_b += p2 + p3;
            split_pair(p0, p1, p_hi[n >> 1][(n & 1) * 2], p_lo[n >> 1][(n & 1) * 2]);
            split_pair(p2, p3, p_hi[n >> 1][(n & 1) * 2 + 1], p_lo[n >> 1][(n & 1) * 2 + 1]);
        }
        l_a = l_a * rescale_a + sum_a;
        l_b = l_b * rescale_b + sum_b;
#pragma unroll
        for (int n = 0; n < VD / 8; ++n) {
            o_acc[n][0] *= rescale_a; o_acc[n][1] *= rescale_a;
            o_acc[n][2] *= rescale_b; o_acc[n][3] *= rescale_b;
        }
#pragma unroll
        for (int kk = 0; kk < TL_BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < VD / 16; dp += 2) {
                // two blocks of 16 dimensions at a time, so that the product with the rest of a weight
                // follows the product with its head on the same accumulator four instructions later, not two
                uint32_t b[4], c[4];
                const int matrix = lane >> 3;
                const int key = kk * 16 + (matrix & 1) * 8 + (lane & 7);
                const int dim = dp * 16 + (matrix >> 1) * 8;
                ldmatrix_x4_trans(b, v_tile + key * VROW + dim);
                if (dp + 1 < VD / 16) ldmatrix_x4_trans(c, v_tile + key * VROW + dim + 16);
                mma_bf16(o_acc[2 * dp], p_hi[kk], b[0], b[1]);
                mma_bf16(o_acc[2 * dp + 1], p_hi[kk], b[2], b[3]);
                if (dp + 1 < VD / 16) {
                    mma_bf16(o_acc[2 * dp + 2], p_hi[kk], c[0], c[1]);
                    mma_bf16(o_acc[2 * dp + 3], p_hi[kk], c[2], c[3]);
                }
                mma_bf16(o_acc[2 * dp], p_lo[kk], b[0], b[1]);
                mma_bf16(o_acc[2 * dp + 1], p_lo[kk], b[2], b[3]);
                if (dp + 1 < VD / 16) {
                    mma_bf16(o_acc[2 * dp + 2], p_lo[kk], c[0], c[1]);
                    mma_bf16(o_acc[2 * dp + 3], p_lo[kk], c[2], c[3]);
                }
            }
        }
    }
    if (!busy) return;

    // ---- the four threads of a row hold partial sums of its denominator
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (SINGLES) {
        // partial (max, sum, out) of this chunk for head row_a / row_b of the group
        const int slots = a.window_chunks + a.kept_chunks;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = half ? row_b : row_a;
            if (row >= count) continue;
            float* dst = a.scratch + (((int64_t)first_token * a.num_q + head0 + row) * slots + blockIdx.z) * (VD + 2);
            if (t4 == 0) { dst[0] = half ? m_b : m_a; dst[1] = half ? l_b : l_a; }
#pragma unroll
            for (int n = 0; n < VD / 8; ++n) {
                const int dim = n * 8 + 2 * t4;
                dst[2 + dim] = o_acc[n][half * 2];
                dst[3 + dim] = o_acc[n][half * 2 + 1];
            }
        }
        return;
    }
    float keep_a = 1.0f, keep_b = 1.0f;
    if (a.sinks) {
        // the sink joins the denominator: exp(sink) beside the keys' exponentials, under a common reference
        const float sink = a.sinks[head0] * TL_LOG2E;
        const float top_a = fmaxf(m_a, sink), top_b = fmaxf(m_b, sink);
        keep_a = exp2f(m_a - top_a);
        keep_b = exp2f(m_b - top_b);
        l_a = l_a * keep_a + exp2f(sink - top_a);
        l_b = l_b * keep_b + exp2f(sink - top_b);
    }
    const float inv_a = keep_a / l_a, inv_b = keep_b / l_b;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int row = half ? row_b : row_a;
        if (row >= count) continue;
        float inv = half ? inv_b : inv_a;
        bf16* dst = a.out + (int64_t)(first_token + row) * a.out_token_stride + (int64_t)head0 * VD;
        const bf16* gate = nullptr;
        if (a.gate && a.gate_per_head)
            inv *= sigmoid_of(__bfloat162float(a.gate[(int64_t)(first_token + row) * a.gate_token_stride + head0]));
        else if (a.gate)
            gate = a.gate + (int64_t)(first_token + row) * a.gate_token_stride + (int64_t)head0 * VD;
#pragma unroll
        for (int n = 0; n < VD / 8; ++n) {
            const int dim = n * 8 + 2 * t4;
            float x = o_acc[n][half * 2] * inv, y = o_acc[n][half * 2 + 1] * inv;
            if (gate) {
                const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + dim));
                x *= sigmoid_of(gv.x);
                y *= sigmoid_of(gv.y);
            }
            *reinterpret_cast<uint32_t*>(dst + dim) = pack_bf16x2(x, y);
        }
    }
}

// Which chunk the CTA with index z of a token takes: z < window_chunks counts back from the token's own
// chunk; the others are the chunks of kept keys that lie wholly before the window's first chunk.
// Returns -1 where there is nothing to do.
__device__ __forceinline__ int chunk_of_slot(int z, int window_chunks, int position, int lo, int kept) {
    const int own = position / TL_CHUNK, first_chunk = lo / TL_CHUNK;
    if (z < window_chunks) {
        const int chunk = own - z;
        return chunk < first_chunk ? -1 : chunk;
    }
    const int chunk = z - window_chunks;
    return (chunk >= first_chunk || chunk * TL_CHUNK >= kept) ? -1 : chunk;
}

// Single tokens, up to 16 q heads a kv head: one chunk of TL_CHUNK keys a CTA, all of it copied in at
// once; warp w takes the keys w * 32 .. w * 32 + 31 of the chunk, the four partial results are merged in
// shared memory in the order of the keys and leave as one (max, sum, out) per head.
template <int KD, int VD>
__global__ void __launch_bounds__(TL_WARPS * 32, 3) attention_singles_kernel(const TileArgs a) {
    constexpr bool VIK = TILES_VALUE_IN_KEY != 0;
    constexpr int KROW = KD + TL_PAD, VROW = VIK ? KROW : VD + TL_PAD;
    constexpr int KCHUNKS = KD / 8, VCHUNKS = VD / 8;
    static_assert(TL_CHUNK == TL_WARPS * TL_BN, "a warp takes one tile of the chunk");
    static_assert(!VIK || VD <= KD, "values inside the key rows are no longer than the rows");
    extern __shared__ __align__(16) unsigned char shared_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(shared_raw);                         // [16][KROW]
    bf16* k_s = q_s + 16 * KROW;                                             // [chunk][KROW]
    bf16* v_s = VIK ? k_s : k_s + TL_CHUNK * KROW;                           // [chunk][VROW], or the keys
    int* slot_s = reinterpret_cast<int*>(VIK ? k_s + TL_CHUNK * KROW : v_s + TL_CHUNK * VROW);   // [chunk]
    float* part_s = reinterpret_cast<float*>(k_s);                           // over K and V once they are used up

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int token = blockIdx.x;
    const int request = a.token_row[token], position = a.positions[token];
    if (request < 0 || position < 0) return;                 // a padding row; the merge writes its zeros
    const int group = a.num_q / a.num_kv, kv_head = blockIdx.y, head0 = kv_head * group;
    const int lo = lowest_seen(a, position);
    const int kept = min(a.keep_first, lo);
    const int chunk = chunk_of_slot(blockIdx.z, a.window_chunks, position, lo, kept);
    if (chunk < 0) return;
    const int key0 = chunk * TL_CHUNK;
    const int* table = a.block_tables + (int64_t)request * a.table_stride;

    {   // where each key of the chunk lies; keys the token does not see are not even fetched
        const int key = key0 + tid;
        int slot = -1;
        if (key <= position && (key >= lo || key < kept)) {
            const int page = table[key / a.page_size];
            if (page >= 0) slot = (page * a.num_kv + kv_head) * a.page_size + key % a.page_size;
        }
        slot_s[tid] = slot;
    }
    for (int index = tid; index < 16 * KCHUNKS; index += TL_WARPS * 32) {
        const int r = index / KCHUNKS, c = index % KCHUNKS;
        cp_async_16(q_s + r * KROW + c * 8,
                    a.q + (int64_t)token * a.q_token_stride + (int64_t)(head0 + min(r, group - 1)) * KD + c * 8, r < group);
    }
    __syncthreads();
    for (int index = tid; index < TL_CHUNK * KCHUNKS; index += TL_WARPS * 32) {
        const int r = index / KCHUNKS, c = index % KCHUNKS;
        const int slot = slot_s[r];
        cp_async_16(k_s + r * KROW + c * 8, a.key_cache + (int64_t)max(slot, 0) * KD + c * 8, slot >= 0);
    }
    if (!VIK) {
        for (int index = tid; index < TL_CHUNK * VCHUNKS; index += TL_WARPS * 32) {
            const int r = index / VCHUNKS, c = index % VCHUNKS;
            const int slot = slot_s[r];
            cp_async_16(v_s + r * VROW + c * 8, a.value_cache + (int64_t)max(slot, 0) * VD + c * 8, slot >= 0);
        }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    const int g = lane >> 2, t4 = lane & 3;
    const int tile_key = key0 + warp * TL_BN;
    const bool any = tile_key <= position && (tile_key + TL_BN - 1 >= lo || tile_key < kept);
    float o_acc[VD / 8][4];
#pragma unroll
    for (int n = 0; n < VD / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) o_acc[n][i] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    if (any) {
        const bf16* k_tile = k_s + warp * TL_BN * KROW;
        const bf16* v_tile = v_s + warp * TL_BN * VROW;
        const bf16* q_lane = q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * KROW + (lane >> 4) * 8;
        float s_acc[TL_BN / 8][4];
#pragma unroll
        for (int n = 0; n < TL_BN / 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) s_acc[n][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KD / 16; ++ks) {
            uint32_t q_frag[4];
            ldmatrix_x4(q_frag, q_lane + ks * 16);
#pragma unroll
            for (int np = 0; np < TL_BN / 16; ++np) {
                uint32_t b[4];
                const int matrix = lane >> 3;
                const int key = np * 16 + (matrix >> 1) * 8 + (lane & 7);
                const int dim = ks * 16 + (matrix & 1) * 8;
                ldmatrix_x4(b, k_tile + key * KROW + dim);
                mma_bf16(s_acc[2 * np], q_frag, b[0], b[1]);
                mma_bf16(s_acc[2 * np + 1], q_frag, b[2], b[3]);
            }
        }
        const float scale_log2 = a.scale * TL_LOG2E;
        const bool biased = a.slopes != nullptr;
        const float slope_a = biased ? a.slopes[head0 + min(g, group - 1)] * TL_LOG2E : 0.0f;
        const float slope_b = biased ? a.slopes[head0 + min(g + 8, group - 1)] * TL_LOG2E : 0.0f;
#pragma unroll
        for (int n = 0; n < TL_BN / 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int key = tile_key + n * 8 + 2 * t4 + (i & 1);
                float s = s_acc[n][i] * scale_log2;
                if (biased) s -= (i < 2 ? slope_a : slope_b) * (float)(position - key);
                if (a.bias_table) s += table_bias(a, position - key, head0 + min(i < 2 ? g : g + 8, group - 1));
                if (!(key <= position && (key >= lo || key < kept))) s = -INFINITY;
                s_acc[n][i] = s;
                if (i < 2) m_a = fmaxf(m_a, s); else m_b = fmaxf(m_b, s);
            }
        }
        m_a = fmaxf(m_a, __shfl_xor_sync(0xffffffffu, m_a, 1));
        m_a = fmaxf(m_a, __shfl_xor_sync(0xffffffffu, m_a, 2));
        m_b = fmaxf(m_b, __shfl_xor_sync(0xffffffffu, m_b, 1));
        m_b = fmaxf(m_b, __shfl_xor_sync(0xffffffffu, m_b, 2));
        uint32_t p_hi[TL_BN / 16][4], p_lo[TL_BN / 16][4];
#pragma unroll
        for (int n = 0; n < TL_BN / 8; ++n) {
            const float p0 = exp2f(s_acc[n][0] - m_a), p1 = exp2f(s_acc[n][1] - m_a);      // the tile has a key every row sees
            const float p2 = exp2f(s_acc[n][2] - m_b), p3 = exp2f(s_acc[n][3] - m_b);
            l_a += p0 + p1;
            l_b += p2 + p3;
            split_pair(p0, p1, p_hi[n >> 1][(n & 1) * 2], p_lo[n >> 1][(n & 1) * 2]);
            split_pair(p2, p3, p_hi[n >> 1][(n & 1) * 2 + 1], p_lo[n >> 1][(n & 1) * 2 + 1]);
        }
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
#pragma unroll
        for (int kk = 0; kk < TL_BN / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < VD / 16; dp += 2) {
                // two blocks of 16 dimensions at a time, so that the product with the rest of a weight
                // follows the product with its head on the same accumulator four instructions later, not two
                uint32_t b[4], c[4];
                const int matrix = lane >> 3;
                const int key = kk * 16 + (matrix & 1) * 8 + (lane & 7);
                const int dim = dp * 16 + (matrix >> 1) * 8;
                ldmatrix_x4_trans(b, v_tile + key * VROW + dim);
                if (dp + 1 < VD / 16) ldmatrix_x4_trans(c, v_tile + key * VROW + dim + 16);
                mma_bf16(o_acc[2 * dp], p_hi[kk], b[0], b[1]);
                mma_bf16(o_acc[2 * dp + 1], p_hi[kk], b[2], b[3]);
                if (dp + 1 < VD / 16) {
                    mma_bf16(o_acc[2 * dp + 2], p_hi[kk], c[0], c[1]);
                    mma_bf16(o_acc[2 * dp + 3], p_hi[kk], c[2], c[3]);
                }
                mma_bf16(o_acc[2 * dp], p_lo[kk], b[0], b[1]);
                mma_bf16(o_acc[2 * dp + 1], p_lo[kk], b[2], b[3]);
                if (dp + 1 < VD / 16) {
                    mma_bf16(o_acc[2 * dp + 2], p_lo[kk], c[0], c[1]);
                    mma_bf16(o_acc[2 * dp + 3], p_lo[kk], c[2], c[3]);
                }
            }
        }
    }
    __syncthreads();                                      // every warp is done with K and V: the partials go there
    float* pm = part_s;                                   // [warps][16]
    float* pl = pm + TL_WARPS * 16;                       // [warps][16]
    float* po = pl + TL_WARPS * 16;                       // [warps][16][VD]
    if (t4 == 0) {
        pm[warp * 16 + g] = m_a; pm[warp * 16 + g + 8] = m_b;
        pl[warp * 16 + g] = l_a; pl[warp * 16 + g + 8] = l_b;
    }
#pragma unroll
    for (int n = 0; n < VD / 8; ++n) {
        const int dim = n * 8 + 2 * t4;
        float* ra = po + ((warp * 16 + g) * VD + dim);
        float* rb = po + ((warp * 16 + g + 8) * VD + dim);
        ra[0] = o_acc[n][0]; ra[1] = o_acc[n][1];
        rb[0] = o_acc[n][2]; rb[1] = o_acc[n][3];
    }
    __syncthreads();
    const int slots = a.window_chunks + a.kept_chunks;
    for (int index = tid; index < group * VD; index += TL_WARPS * 32) {
        const int row = index / VD, dim = index % VD;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < TL_WARPS; ++w) top = fmaxf(top, pm[w * 16 + row]);
        float sum = 0.0f, out = 0.0f;
#pragma unroll
        for (int w = 0; w < TL_WARPS; ++w) {
            const float m = pm[w * 16 + row];
            const float weight = m == -INFINITY ? 0.0f : exp2f(m - top);
            sum += pl[w * 16 + row] * weight;
            out += po[(w * 16 + row) * VD + dim] * weight;
        }
        float* dst = a.scratch + (((int64_t)token * a.num_q + head0 + row) * slots + blockIdx.z) * (VD + 2);
        if (dim == 0) { dst[0] = top; dst[1] = sum; }
        dst[2 + dim] = out;
    }
}

// One warp per (token, head): the partial results of the row's chunks, in ascending order of their keys
// (kept first keys, then the window from its oldest chunk to the token's own), divided, gated, stored.
// The largest maximum is found first, so that the sums do not wait for one another.
template <int VD>
__global__ void merge_singles_kernel(const TileArgs a, int tokens) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * TL_WARPS + warp;
    if (row >= (int64_t)tokens * a.num_q) return;
    const int token = (int)(row / a.num_q), head = (int)(row % a.num_q);
    const int position = a.positions[token];
    bf16* dst = a.out + (int64_t)token * a.out_token_stride + (int64_t)head * VD;
    if (a.token_row[token] < 0 || position < 0) {
        for (int dim = lane; dim < VD; dim += 32) dst[dim] = __float2bfloat16_rn(0.0f);
        return;
    }
    const int lo = lowest_seen(a, position);
    const int kept = min(a.keep_first, lo);
    const int own = position / TL_CHUNK, first_chunk = lo / TL_CHUNK;
    const int slots = a.window_chunks + a.kept_chunks;
    const float* base = a.scratch + row * slots * (int64_t)(VD + 2);
    // the row's slots in ascending key order: n_kept chunks of kept keys, then own - first_chunk + 1 of the window
    const int n_kept = min(min(first_chunk, a.kept_chunks), (kept + TL_CHUNK - 1) / TL_CHUNK);
    const int n_window = own - first_chunk + 1;
    auto slot_of = [&](int i) { return i < n_kept ? a.window_chunks + i : n_window - 1 - (i - n_kept); };
    const int count = n_kept + n_window;
    float top = -INFINITY;
    for (int i = lane; i < count; i += 32) top = fmaxf(top, base[(int64_t)slot_of(i) * (VD + 2)]);
    top = warp_max(top);
    constexpr int PER = (VD + 31) / 32;
    float l = 0.0f, o[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) o[i] = 0.0f;
#pragma unroll 4
    for (int i = 0; i < count; ++i) {
        const float* src = base + (int64_t)slot_of(i) * (VD + 2);
        const float m = src[0];
        const float weight = m == -INFINITY ? 0.0f : exp2f(m - top);
        l += src[1] * weight;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int dim = lane + 32 * j;
            if (dim < VD) o[j] += src[2 + dim] * weight;
        }
    }
    float keep = 1.0f;
    if (a.sinks) {
        const float sink = a.sinks[head] * TL_LOG2E;
        const float both = fmaxf(top, sink);
        keep = exp2f(top - both);
        l = l * keep + exp2f(sink - both);
    }
    float inv = keep / l;
    const bf16* gate = nullptr;
    if (a.gate && a.gate_per_head) inv *= sigmoid_of(__bfloat162float(a.gate[(int64_t)token * a.gate_token_stride + head]));
    else if (a.gate) gate = a.gate + (int64_t)token * a.gate_token_stride + (int64_t)head * VD;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int dim = lane + 32 * i;
        if (dim < VD) {
            float x = o[i] * inv;
            if (gate) x *= sigmoid_of(__bfloat162float(gate[dim]));
            dst[dim] = __float2bfloat16_rn(x);
        }
    }
}

extern "C" int tvb_attention_tiles_key_dim() { return TILES_KEY_DIM; }
extern "C" int tvb_attention_tiles_value_dim() { return TILES_VALUE_DIM; }
extern "C" int tvb_attention_tiles_tile_tokens() { return TL_BM; }
extern "C" int tvb_attention_tiles_chunk_keys() { return TL_CHUNK; }

extern "C" int tvb_attention_tiles_value_in_key() { return TILES_VALUE_IN_KEY; }

static size_t tiles_shared_bytes() {
    return (size_t)(TL_BM + 2 * TL_BN) * (TILES_KEY_DIM + TL_PAD) * sizeof(bf16) +
           (TILES_VALUE_IN_KEY ? 0 : (size_t)2 * TL_BN * (TILES_VALUE_DIM + TL_PAD) * sizeof(bf16)) +
           2 * TL_BN * sizeof(int);
}

static int check_common(const TileArgs& a, int key_dim, int value_dim) {
    if (a.segment < 0 || (a.segment > 0 && a.window > 0) || (a.bias_table && a.bias_rows <= 0)) return TVB_BAD_ARGUMENT;
    if (key_dim != TILES_KEY_DIM || value_dim != TILES_VALUE_DIM || TILES_KEY_DIM % 16 || TILES_VALUE_DIM % 16 ||
        a.num_q <= 0 || a.num_kv <= 0 || a.num_q % a.num_kv || a.page_size <= 0 || a.window < 0 || a.keep_first < 0 ||
        (a.q_token_stride * 2) % 16 || ((uintptr_t)a.q) % 16 || a.out_token_stride % 2 || ((uintptr_t)a.out) % 4 ||
        (a.gate && !a.gate_per_head && (a.gate_token_stride % 2 || ((uintptr_t)a.gate) % 4)) ||
        (!TILES_VALUE_IN_KEY && !a.value_cache) || (TILES_VALUE_IN_KEY && TILES_VALUE_DIM > TILES_KEY_DIM))
        return TVB_BAD_ARGUMENT;
    return 0;
}

// Prompt portions: tile i holds tile_count[i] (1..64) consecutive tokens from flat index tile_first[i]
// on, of the request in row tile_row[i] of block_tables.
// `slopes` and `sinks`: float32 [num_q] or null; `gate_per_head`: the gate holds one number a head.
// `bias_table`: float32 [bias_rows, num_q] or null; `segment`: 0 for none.
extern "C" int tvb_attention_tiles_table(const void* q, long long q_token_stride, const void* key_cache,
                                         const void* value_cache, const int* block_tables, int table_stride,
                                         const int* positions, const int* tile_row, const int* tile_first,
                                         const int* tile_count, void* out, long long out_token_stride,
                                         const void* gate, long long gate_token_stride, int gate_per_head,
                                         const float* slopes, const float* sinks, const float* bias_table,
                                         int bias_rows, int segment, int tiles, int num_q, int num_kv,
                                         int key_dim, int value_dim, int page_size, int window, int keep_first,
                                         float scale, void* stream) {
    if (tiles <= 0) return 0;
    TileArgs a{(const bf16*)q, q_token_stride, (const bf16*)key_cache, (const bf16*)value_cache, block_tables,
               table_stride, positions, nullptr, tile_row, tile_first, tile_count, (bf16*)out, out_token_stride,
               (const bf16*)gate, gate_token_stride, nullptr, 0, 0, num_q, num_kv, page_size, window,
               window > 0 ? keep_first : 0, scale, slopes, sinks, gate_per_head, bias_table, bias_rows, segment};
    if (check_common(a, key_dim, value_dim) || num_q > 65535) return TVB_BAD_ARGUMENT;
    auto kernel = attention_tiles_kernel<TILES_KEY_DIM, TILES_VALUE_DIM, false>;
    const size_t shared = tiles_shared_bytes();
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (e != cudaSuccess) return (int)e;
    kernel<<<dim3(tiles, num_q), TL_WARPS * 32, shared, (cudaStream_t)stream>>>(a);
    return tvb_last_error();
}

extern "C" int tvb_attention_tiles_biased(const void* q, long long q_token_stride, const void* key_cache,
                                          const void* value_cache, const int* block_tables, int table_stride,
                                          const int* positions, const int* tile_row, const int* tile_first,
                                          const int* tile_count, void* out, long long out_token_stride,
                                          const void* gate, long long gate_token_stride, int gate_per_head,
                                          const float* slopes, const float* sinks, int tiles, int num_q, int num_kv,
                                          int key_dim, int value_dim, int page_size, int window, int keep_first,
                                          float scale, void* stream) {
    return tvb_attention_tiles_table(q, q_token_stride, key_cache, value_cache, block_tables, table_stride, positions,
                                     tile_row, tile_first, tile_count, out, out_token_stride, gate, gate_token_stride,
                                     gate_per_head, slopes, sinks, nullptr, 0, 0, tiles, num_q, num_kv, key_dim,
                                     value_dim, page_size, window, keep_first, scale, stream);
}

extern "C" int tvb_attention_tiles(const void* q, long long q_token_stride, const void* key_cache,
                                   const void* value_cache, const int* block_tables, int table_stride,
                                   const int* positions, const int* tile_row, const int* tile_first,
                                   const int* tile_count, void* out, long long out_token_stride, const void* gate,
                                   long long gate_token_stride, int tiles, int num_q, int num_kv, int key_dim,
                                   int value_dim, int page_size, int window, int keep_first, float scale,
                                   void* stream) {
    return tvb_attention_tiles_biased(q, q_token_stride, key_cache, value_cache, block_tables, table_stride, positions,
                                      tile_row, tile_first, tile_count, out, out_token_stride, gate, gate_token_stride,
                                      0, nullptr, nullptr, tiles, num_q, num_kv, key_dim, value_dim, page_size, window,
                                      keep_first, scale, stream);
}

// How many chunk slots a row of the singles form has: (for the window, for kept first keys).
static void singles_chunks(int window, int keep_first, int max_context, int* window_chunks, int* kept_chunks) {
    const int all = (max_context + TL_CHUNK - 1) / TL_CHUNK;
    if (window <= 0) { *window_chunks = all > 0 ? all : 1; *kept_chunks = 0; return; }
    const int spanned = (window + TL_CHUNK - 2) / TL_CHUNK + 1;       // chunks a window can touch
    *window_chunks = spanned < all ? spanned : (all > 0 ? all : 1);
    *kept_chunks = (keep_first + TL_CHUNK - 1) / TL_CHUNK;
}

// `window`: with segments, the segment's size (a segment touches the chunks a window of its size can).
extern "C" long long tvb_attention_tiles_singles_floats(int tokens, int num_q, int window, int keep_first,
                                                         int max_context) {
    int wc, kc;
    singles_chunks(window, window > 0 ? keep_first : 0, max_context, &wc, &kc);
    return (long long)tokens * num_q * (wc + kc) * (TILES_VALUE_DIM + 2);
}

// Single tokens (decoded ones): token i is of the request in row token_row[i] (-1: padding) at
// positions[i] < max_context; its keys and values are in the cache already.
extern "C" int tvb_attention_tiles_singles_table(const void* q, long long q_token_stride, const void* key_cache,
                                                 const void* value_cache, const int* block_tables, int table_stride,
                                                 const int* positions, const int* token_row, void* out,
                                                 long long out_token_stride, const void* gate,
                                                 long long gate_token_stride, int gate_per_head, const float* slopes,
                                                 const float* sinks, const float* bias_table, int bias_rows,
                                                 int segment, float* scratch, int tokens, int num_q,
                                                 int num_kv, int key_dim, int value_dim, int page_size, int window,
                                                 int keep_first, float scale, int max_context, void* stream) {
    if (tokens <= 0) return 0;
    TileArgs a{(const bf16*)q, q_token_stride, (const bf16*)key_cache, (const bf16*)value_cache, block_tables,
               table_stride, positions, token_row, nullptr, nullptr, nullptr, (bf16*)out, out_token_stride,
               (const bf16*)gate, gate_token_stride, scratch, 0, 0, num_q, num_kv, page_size, window,
               window > 0 ? keep_first : 0, scale, slopes, sinks, gate_per_head, bias_table, bias_rows, segment};
    if (check_common(a, key_dim, value_dim) || !scratch || max_context <= 0 || num_q / num_kv > TL_BM || num_kv > 65535)
        return TVB_BAD_ARGUMENT;
    singles_chunks(a.segment > 0 ? a.segment : a.window, a.keep_first, max_context, &a.window_chunks, &a.kept_chunks);
    if (a.window_chunks + a.kept_chunks > 65535) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(tokens, num_kv, a.window_chunks + a.kept_chunks);
    if (num_q / num_kv <= 16) {
        auto kernel = attention_singles_kernel<TILES_KEY_DIM, TILES_VALUE_DIM>;
        const size_t shared = (size_t)(16 + TL_CHUNK) * (TILES_KEY_DIM + TL_PAD) * sizeof(bf16) +
                              (TILES_VALUE_IN_KEY ? 0 : (size_t)TL_CHUNK * (TILES_VALUE_DIM + TL_PAD) * sizeof(bf16)) +
                              TL_CHUNK * sizeof(int);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, TL_WARPS * 32, shared, s>>>(a);
    } else {
        auto kernel = attention_tiles_kernel<TILES_KEY_DIM, TILES_VALUE_DIM, true>;
        const size_t shared = tiles_shared_bytes();
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (e != cudaSuccess) return (int)e;
        kernel<<<grid, TL_WARPS * 32, shared, s>>>(a);
    }
    const int64_t rows = (int64_t)tokens * num_q;
    merge_singles_kernel<TILES_VALUE_DIM><<<(unsigned)((rows + TL_WARPS - 1) / TL_WARPS), TL_WARPS * 32, 0, s>>>(a, tokens);
    return tvb_last_error();
}

extern "C" int tvb_attention_tiles_singles_biased(const void* q, long long q_token_stride, const void* key_cache,
                                                  const void* value_cache, const int* block_tables, int table_stride,
                                                  const int* positions, const int* token_row, void* out,
                                                  long long out_token_stride, const void* gate,
                                                  long long gate_token_stride, int gate_per_head, const float* slopes,
                                                  const float* sinks, float* scratch, int tokens, int num_q,
                                                  int num_kv, int key_dim, int value_dim, int page_size, int window,
                                                  int keep_first, float scale, int max_context, void* stream) {
    return tvb_attention_tiles_singles_table(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                                             positions, token_row, out, out_token_stride, gate, gate_token_stride,
                                             gate_per_head, slopes, sinks, nullptr, 0, 0, scratch, tokens, num_q,
                                             num_kv, key_dim, value_dim, page_size, window, keep_first, scale,
                                             max_context, stream);
}

extern "C" int tvb_attention_tiles_singles(const void* q, long long q_token_stride, const void* key_cache,
                                           const void* value_cache, const int* block_tables, int table_stride,
                                           const int* positions, const int* token_row, void* out,
                                           long long out_token_stride, const void* gate, long long gate_token_stride,
                                           float* scratch, int tokens, int num_q, int num_kv, int key_dim,
                                           int value_dim, int page_size, int window, int keep_first, float scale,
                                           int max_context, void* stream) {
    return tvb_attention_tiles_singles_biased(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                                              positions, token_row, out, out_token_stride, gate, gate_token_stride, 0,
                                              nullptr, nullptr, scratch, tokens, num_q, num_kv, key_dim, value_dim,
                                              page_size, window, keep_first, scale, max_context, stream);
}
