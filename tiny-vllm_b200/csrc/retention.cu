// Retention: linear attention with a fixed decay a head, no softmax and no denominator.
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T          (a state [dim, vdim] a head and request, float32)
//   o_t = S_t^T q_t
//
// Three kernels between a mixer's input and output projections:
//
//   retention_prepare   q and k heads of the packed projection -> float32 rows, the first `rot_dims`
//                       dimensions of every head turned by position * inv_freq (pairs (i, i + rot/2)
//                       or (2i, 2i + 1)), k then multiplied by `key_scale`
//   retention_scan      the recurrence itself, token by token from the state the request's earlier
//                       tokens left (a slot of the state arena) to the state its next tokens start
//                       from (or, for long prompts, in pieces side by side that a second kernel joins and
//                       a third corrects); a CTA has one (request or piece, head, block of value columns),
//                       a thread up to eight rows by eight columns of the state in registers; tokens come
//                       in blocks of four through
//                       shared memory, the next block's loads in flight while this one is computed
//   retention_finish    every head's o divided by its root mean square (or not), times act(gate),
//                       rounded once to the storage type
//
// Angles, the rotated q and k, the outer products, the state and the sums are float32 whatever the
// storage type; only v and the gate are read in it and only the finished output is rounded to it.
#include "common.cuh"

// RET_GATED (a macro, a library each): 0, the form above; 1, a decay a token and key channel instead of one a
// head, read from `gates` [tokens, heads * dim] (float32), with the keys tied to it, k = 1 - gate:
//   S_t = diag(g_t) S_(t-1) + (1 - g_t) v_t^T
// (a channel writes with the strength it does not keep); 2, such decays beside keys of their own.  In the pieces
// form the decay of a piece is the product of its tokens' gates, channel by channel, and the correcting pass
// reads queries that a kernel of its own multiplied by the running products.
#ifndef RET_GATED
#define RET_GATED 0
#endif

#define RET_PAIR_INTERLEAVED 0
#define RET_PAIR_HALF_SPLIT 1
#define RET_MAX_TURNED 512        // pairs of a head that turn: sine and cosine of a token in shared memory

template <typename T>
__global__ void __launch_bounds__(128) retention_prepare_kernel(
    const T* __restrict__ proj, int64_t token_stride, int q_at, int k_at, int heads, int dim,
    const float* __restrict__ inv_freq, int rot_dims, int pairing, float key_scale,
    const int* __restrict__ positions, float* __restrict__ q_out, float* __restrict__ k_out) {
    __shared__ float cos_s[RET_MAX_TURNED], sin_s[RET_MAX_TURNED];
    const int token = blockIdx.x;                 // block y: a slice of the row's q and k elements
    const int half = inv_freq ? rot_dims >> 1 : 0;
    const float position = (float)max(positions[token], 0);
    for (int j = threadIdx.x; j < half; j += blockDim.x)
        sincosf(__fmul_rn(position, inv_freq[j]), &sin_s[j], &cos_s[j]);
    __syncthreads();
    const T* row = proj + (int64_t)token * token_stride;
    const int per = heads * dim;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < 2 * per; e += gridDim.y * blockDim.x) {
        const bool is_key = e >= per;
        const int inside = is_key ? e - per : e;
        const int i = inside % dim;
        const T* src = row + (is_key ? k_at : q_at) + inside - i;        // the head's first element
        float x = to_float<T>(src[i]);
        if (i < 2 * half) {
            int pair, other;
            bool first;
            if (pairing == RET_PAIR_HALF_SPLIT) { first = i < half; pair = first ? i : i - half; other = first ? i + half : i - half; }
            else { first = (i & 1) == 0; pair = i >> 1; other = first ? i + 1 : i - 1; }
            const float y = to_float<T>(src[other]);
            const float c = cos_s[pair], s = sin_s[pair];
            x = first ? __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)) : __fadd_rn(__fmul_rn(x, c), __fmul_rn(y, s));
        }
        if (is_key) k_out[(int64_t)token * per + inside] = __fmul_rn(x, key_scale);
        else q_out[(int64_t)token * per + inside] = x;
    }
}

#define RET_THREADS 128
#define RET_BLOCK 4                               // tokens that wait in shared memory
#define RET_TILE 8                                // value columns a thread
#define RET_SUMS (RET_BLOCK * RET_TILE)           // sums a thread holds after a block of tokens

// A thread holds ROWS rows by RET_TILE columns of the state: rows 4 (group + GROUPS j) .. + 3 for
// j = 0 .. ROWS / 4 - 1 (dim <= GROUPS * ROWS), so that the GROUPS lanes of a tile of columns read
// neighbouring float4s of a token's q and k; a CTA has RET_THREADS / GROUPS tiles of columns.  A token costs a
// thread ROWS / 2 + 2 float4s from shared memory for 3 * ROWS * RET_TILE multiply-adds, which keeps the
// arithmetic, not the shared memory, the busier of the two.  The lanes' partial sums of a block of tokens are
// added by halving: at every step a lane hands half of its sums to the lane one bit away and keeps the
// other half, so that after log2(GROUPS) steps lane g holds sums g * RET_SUMS / GROUPS and on, complete.
template <typename T, int GROUPS, int ROWS, bool CORRECT>
__global__ void __launch_bounds__(RET_THREADS) retention_scan_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ gates,
    const T* __restrict__ v, int64_t v_stride,
    float* __restrict__ state, const float* __restrict__ decay, const int* __restrict__ row_starts,
    const int* __restrict__ state_slots, const int* __restrict__ token_row, float* __restrict__ out,
    float* __restrict__ parts, int segment, int rows, int heads, int dim, int vdim) {
    constexpr int COLS = RET_THREADS / GROUPS * RET_TILE;                   // value columns a CTA
    constexpr int WIDTH = GROUPS * ROWS;
    constexpr int LOADS = (RET_BLOCK * WIDTH + RET_THREADS - 1) / RET_THREADS;  // q (and k) values a thread fetches a block
    constexpr int V_LOADS = RET_BLOCK * COLS / RET_THREADS;
    constexpr int LEFT = RET_SUMS / GROUPS;                                 // sums a lane ends with
    static_assert(ROWS % 4 == 0 && RET_SUMS % GROUPS == 0 && RET_BLOCK * COLS % RET_THREADS == 0, "retention_scan: tile");
    __shared__ __align__(16) float q_s[RET_BLOCK][WIDTH];
    constexpr bool KEYS = !CORRECT && RET_GATED != 1;        // keys of their own wait in shared memory
    constexpr bool GATES = !CORRECT && RET_GATED != 0;       // a decay a token and channel does
    __shared__ __align__(16) float k_s[KEYS ? RET_BLOCK : 1][KEYS ? WIDTH : 4];
    __shared__ __align__(16) float g_s[GATES ? RET_BLOCK : 1][GATES ? WIDTH : 4];
    __shared__ __align__(16) float v_s[CORRECT ? 1 : RET_BLOCK][CORRECT ? 4 : COLS];
    __shared__ float power_s[2][RET_BLOCK];    // decay^(t + 1) of this block's tokens and of the next's
    const int head = blockIdx.y, col0 = blockIdx.z * COLS;
    const int tid = threadIdx.x, group = tid % GROUPS, tile = tid / GROUPS;
    // whole entries (segment == 0: block x is the entry) or pieces of `segment` tokens (block x is the
    // piece, counted through the entries in order)
    int row = blockIdx.x, begin, count;
    if (segment <= 0) {
        begin = row_starts[row];
        count = row_starts[row + 1] - begin;
    } else {
        int before = 0, tokens = 0;
        for (row = 0; row < rows; ++row) {
            tokens = row_starts[row + 1] - row_starts[row];
            const int pieces = (tokens + segment - 1) / segment;
            if ((int)blockIdx.x < before + pieces) break;
            before += pieces;
        }
        if (row == rows) return;                  // the grid is as large as the pieces can be many
        const int piece = blockIdx.x - before;
        begin = row_starts[row] + piece * segment;
        count = min(segment, tokens - piece * segment);
    }
    if (count <= 0) return;
    const int c = col0 + tile * RET_TILE;         // the thread's first column
    const int64_t out_stride = (int64_t)heads * vdim;
    if (token_row[begin] < 0) {                   // a padding row of a recorded batch: no request, no state
        if (!CORRECT && group == 0)
            for (int t = 0; t < count; ++t)
                for (int cc = 0; cc < RET_TILE; ++cc)
                    if (c + cc < vdim) out[(int64_t)(begin + t) * out_stride + (int64_t)head * vdim + c + cc] = 0.0f;
        return;
    }
    const float a = RET_GATED ? 1.0f : decay[head];
    // whole entries start from and leave the request's state; a piece starts from nothing and leaves what
    // its tokens add (`parts`), which the combine kernel turns into the state the piece starts from: the
    // correcting pass reads that and adds what it gives to every token of the piece
    float* mine = (segment <= 0 ? state + (((int64_t)state_slots[row] * heads + head) * dim) * vdim
                                : parts + (((int64_t)blockIdx.x * heads + head) * dim) * vdim) + c;
    // then a float4 of a row of the state is whole and aligned
    const bool by_four = (vdim & 3) == 0 && ((reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(parts)) & 15) == 0;
    float s[ROWS][RET_TILE];
    bool any = false;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int d = 4 * (group + GROUPS * (i >> 2)) + (i & 3);
#pragma unroll
        for (int cc = 0; cc < RET_TILE; ++cc) s[i][cc] = 0.0f;
        if (d < dim && (segment <= 0 || CORRECT)) {
            const float* from = mine + (int64_t)d * vdim;
            if (by_four) {
#pragma unroll
                for (int h = 0; h < RET_TILE / 4; ++h)
                    if (c + 4 * h < vdim) {
                        const float4 x = *reinterpret_cast<const float4*>(from + 4 * h);
                        s[i][4 * h] = x.x; s[i][4 * h + 1] = x.y; s[i][4 * h + 2] = x.z; s[i][4 * h + 3] = x.w;
                    }
            } else {
#pragma unroll
                for (int cc = 0; cc < RET_TILE; ++cc)
                    if (c + cc < vdim) s[i][cc] = from[cc];
            }
#pragma unroll
            for (int cc = 0; cc < RET_TILE; ++cc) any = any || s[i][cc] != 0.0f;
        }
    }
    if (CORRECT && !__syncthreads_or(any)) return;            // the request's first piece: nothing came before
    const int64_t qk_stride = (int64_t)heads * dim;
    const float* q_head = q + (int64_t)begin * qk_stride + (int64_t)head * dim;
    const float* k_head = KEYS ? k + (int64_t)begin * qk_stride + (int64_t)head * dim : nullptr;
    const float* g_head = GATES ? gates + (int64_t)begin * qk_stride + (int64_t)head * dim : nullptr;
    const T* v_head = v + (int64_t)begin * v_stride + (int64_t)head * vdim + col0;
    float q_next[LOADS], k_next[KEYS ? LOADS : 1], g_next[GATES ? LOADS : 1], v_next[V_LOADS];

    auto fetch = [&](int first) {                 // tokens first .. first + RET_BLOCK - 1 into registers
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int e = tid + RET_THREADS * j, t = e / WIDTH, d = e % WIDTH;
            const bool ok = e < RET_BLOCK * WIDTH && first + t < count && d < dim;
            q_next[j] = ok ? q_head[(int64_t)(first + t) * qk_stride + d] : 0.0f;
            if constexpr (KEYS) k_next[j] = ok ? k_head[(int64_t)(first + t) * qk_stride + d] : 0.0f;
            if constexpr (GATES) g_next[j] = ok ? g_head[(int64_t)(first + t) * qk_stride + d] : 0.0f;
        }
        if constexpr (!CORRECT) {
#pragma unroll
            for (int j = 0; j < V_LOADS; ++j) {
                const int e = tid + RET_THREADS * j, t = e / COLS, cc = e % COLS;
                const bool ok = first + t < count && col0 + cc < vdim;
                v_next[j] = ok ? to_float<T>(v_head[(int64_t)(first + t) * v_stride + cc]) : 0.0f;
            }
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int e = tid + RET_THREADS * j;
            if (e < RET_BLOCK * WIDTH) {
                q_s[e / WIDTH][e % WIDTH] = q_next[j];
                if constexpr (KEYS) k_s[e / WIDTH][e % WIDTH] = k_next[j];
                if constexpr (GATES) g_s[e / WIDTH][e % WIDTH] = g_next[j];
            }
        }
        if constexpr (!CORRECT) {
#pragma unroll
            for (int j = 0; j < V_LOADS; ++j) {
                const int e = tid + RET_THREADS * j;
                v_s[e / COLS][e % COLS] = v_next[j];
            }
        }
    };

    fetch(0);
    if (CORRECT && !RET_GATED && tid < RET_BLOCK) power_s[0][tid] = powf(a, (float)(tid + 1));
    for (int first = 0; first < count; first += RET_BLOCK) {
        const int turn = (first / RET_BLOCK) & 1;
        __syncthreads();                          // the block before is read
        stage();
        __syncthreads();
        if (first + RET_BLOCK < count) fetch(first + RET_BLOCK);
        if (CORRECT && !RET_GATED && tid < RET_BLOCK) power_s[turn ^ 1][tid] = powf(a, (float)(first + RET_BLOCK + tid + 1));
        const int here = min(RET_BLOCK, count - first);
        float sums[RET_SUMS];
#pragma unroll
        for (int t = 0; t < RET_BLOCK; ++t) {
#pragma unroll
            for (int cc = 0; cc < RET_TILE; ++cc) sums[t * RET_TILE + cc] = 0.0f;
            if (t < here) {                       // the state moves in the order of the tokens, and only by real ones
                float vv[RET_TILE];
                if constexpr (!CORRECT) {
#pragma unroll
                    for (int h = 0; h < RET_TILE / 4; ++h) {
                        const float4 x = *reinterpret_cast<const float4*>(&v_s[t][tile * RET_TILE + 4 * h]);
                        vv[4 * h] = x.x; vv[4 * h + 1] = x.y; vv[4 * h + 2] = x.z; vv[4 * h + 3] = x.w;
                    }
                }
#pragma unroll
                for (int j = 0; j < ROWS / 4; ++j) {
                    const float4 qq = *reinterpret_cast<const float4*>(&q_s[t][4 * (group + GROUPS * j)]);
                    const float qr[4] = {qq.x, qq.y, qq.z, qq.w};
                    if constexpr (!CORRECT) {
                        float kr[4], gr[4] = {a, a, a, a};
                        if constexpr (GATES) {
                            const float4 gg = *reinterpret_cast<const float4*>(&g_s[t][4 * (group + GROUPS * j)]);
                            gr[0] = gg.x; gr[1] = gg.y; gr[2] = gg.z; gr[3] = gg.w;
                        }
                        if constexpr (KEYS) {
                            const float4 kk = *reinterpret_cast<const float4*>(&k_s[t][4 * (group + GROUPS * j)]);
                            kr[0] = kk.x; kr[1] = kk.y; kr[2] = kk.z; kr[3] = kk.w;
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) kr[i] = __fsub_rn(1.0f, gr[i]);      // what is not kept is written
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int cc = 0; cc < RET_TILE; ++cc)
                                s[4 * j + i][cc] = __fmaf_rn(kr[i], vv[cc], __fmul_rn(gr[i], s[4 * j + i][cc]));
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int cc = 0; cc < RET_TILE; ++cc)
                            sums[t * RET_TILE + cc] = __fmaf_rn(s[4 * j + i][cc], qr[i], sums[t * RET_TILE + cc]);
                }
            }
        }
        // halving: with n sums left, the lanes whose bit is set keep the upper n / 2 and hand over the lower
#pragma unroll
        for (int bit = GROUPS / 2, n = RET_SUMS; bit >= 1; bit >>= 1, n >>= 1) {
            const bool upper = (group & bit) != 0;
#pragma unroll
            for (int i = 0; i < n / 2; ++i) {
                const float hand = upper ? sums[i] : sums[i + n / 2];
                const float keep = upper ? sums[i + n / 2] : sums[i];
                sums[i] = keep + __shfl_xor_sync(0xffffffffu, hand, bit);
            }
        }
#pragma unroll
        for (int i = 0; i < LEFT; ++i) {          // sum group * LEFT + i is token (index / RET_TILE), column (index % RET_TILE)
            const int index = group * LEFT + i, t = index / RET_TILE, cc = index % RET_TILE;
            if (t < here && c + cc < vdim) {
                float* o = out + (int64_t)(begin + first + t) * out_stride + (int64_t)head * vdim + c + cc;
                // decay^(t + 1) S_0^T q_t; with gates the queries came multiplied by the running products
                *o = CORRECT ? (RET_GATED ? __fadd_rn(*o, sums[i]) : __fmaf_rn(power_s[turn][t], sums[i], *o)) : sums[i];
            }
        }
    }
    if constexpr (!CORRECT) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int d = 4 * (group + GROUPS * (i >> 2)) + (i & 3);
            if (d < dim) {
                float* to = mine + (int64_t)d * vdim;
                if (by_four) {
#pragma unroll
                    for (int h = 0; h < RET_TILE / 4; ++h)
                        if (c + 4 * h < vdim)
                            *reinterpret_cast<float4*>(to + 4 * h) =
                                make_float4(s[i][4 * h], s[i][4 * h + 1], s[i][4 * h + 2], s[i][4 * h + 3]);
                } else {
#pragma unroll
                    for (int cc = 0; cc < RET_TILE; ++cc)
                        if (c + cc < vdim) to[cc] = s[i][cc];
                }
            }
        }
    }
}

// The states the pieces of an entry start from.  parts[piece] holds what the piece's tokens add to a state
// of zero; with n the piece's tokens, S_next = decay^n S + parts[piece].  A thread walks one element of the
// state through the entry's pieces, leaves in parts[piece] the state the piece starts from, and in the
// request's slot the state after the entry's last token.
template <int VEC>                                // elements a thread: 4 (float4s, where rows of 4 fit) or 1
__global__ void __launch_bounds__(256) retention_combine_kernel(
    float* __restrict__ state, float* __restrict__ parts, const float* __restrict__ decay,
    const float* __restrict__ piece_gates, const int* __restrict__ row_starts, const int* __restrict__ state_slots,
    const int* __restrict__ token_row, int segment, int heads, int per, int vdim) {
    const int row = blockIdx.z, head = blockIdx.y, e = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (e >= per) return;
    int before = 0;
    for (int r = 0; r < row; ++r) before += (row_starts[r + 1] - row_starts[r] + segment - 1) / segment;
    const int begin = row_starts[row], tokens = row_starts[row + 1] - begin;
    if (tokens <= 0 || token_row[begin] < 0) return;
    const int pieces = (tokens + segment - 1) / segment;
#if RET_GATED
    // the decay of a piece: the product of its tokens' gates in this element's key channel (VEC elements lie in
    // one row of the state)
    const int dim = per / vdim;
    const float* gate_of = piece_gates + ((int64_t)before * heads + head) * dim + e / vdim;
    const int64_t gates_apart = (int64_t)heads * dim;
#else
    const float a = decay[head];
    const float whole = powf(a, (float)segment);
    const float rest = powf(a, (float)(tokens - (pieces - 1) * segment));      // the last piece may be shorter
#endif
    float* mine = state + ((int64_t)state_slots[row] * heads + head) * per + e;
    float* first = parts + ((int64_t)before * heads + head) * per + e;
    const int64_t apart = (int64_t)heads * per;
    float s[VEC];
    auto load = [&](const float* p, float* x) {
        if constexpr (VEC == 4) { const float4 y = *reinterpret_cast<const float4*>(p); x[0] = y.x; x[1] = y.y; x[2] = y.z; x[3] = y.w; }
        else x[0] = *p;
    };
    auto store = [&](float* p, const float* x) {
        if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
        else *p = x[0];
    };
    load(mine, s);
    for (int j0 = 0; j0 < pieces; j0 += 8) {      // eight pieces' loads are in flight together
        float added[8][VEC];
#if RET_GATED
        float powers[8];
#endif
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (j0 + u < pieces) {
                load(first + (j0 + u) * apart, added[u]);
#if RET_GATED
                powers[u] = gate_of[(j0 + u) * gates_apart];
#endif
            }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (j0 + u >= pieces) break;
            store(first + (j0 + u) * apart, s);
#if RET_GATED
            const float power = powers[u];
#else
            const float power = j0 + u == pieces - 1 ? rest : whole;
#endif
#pragma unroll
            for (int i = 0; i < VEC; ++i) s[i] = __fmaf_rn(power, s[i], added[u][i]);
        }
    }
    store(mine, s);
}

// With a decay a token and channel: the running product of a piece's gates, channel by channel.  A thread walks
// one channel of one head through one piece, leaves q_t times the product up to and with token t (what the
// correcting pass multiplies with the state the piece starts from) and, at the end, the piece's whole product.
__global__ void __launch_bounds__(128) retention_gate_prefix_kernel(
    const float* __restrict__ q, const float* __restrict__ gates, float* __restrict__ scaled_q,
    float* __restrict__ piece_gates, const int* __restrict__ row_starts, const int* __restrict__ token_row,
    int segment, int rows, int heads, int dim) {
    const int head = blockIdx.y;
    int row, before = 0, tokens = 0;
    for (row = 0; row < rows; ++row) {
        tokens = row_starts[row + 1] - row_starts[row];
        const int pieces = (tokens + segment - 1) / segment;
        if ((int)blockIdx.x < before + pieces) break;
        before += pieces;
    }
    if (row == rows) return;
    const int piece = blockIdx.x - before;
    const int begin = row_starts[row] + piece * segment;
    const int count = min(segment, tokens - piece * segment);
    if (count <= 0 || token_row[begin] < 0) return;
    const int64_t stride = (int64_t)heads * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        const int64_t at = (int64_t)begin * stride + (int64_t)head * dim + d;
        float product = 1.0f;
        for (int t0 = 0; t0 < count; t0 += 8) {           // eight tokens' loads are in flight together
            float g[8], x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (t0 + u < count) { g[u] = gates[at + (t0 + u) * stride]; x[u] = q[at + (t0 + u) * stride]; }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (t0 + u < count) {
                    product = __fmul_rn(product, g[u]);
                    scaled_q[at + (t0 + u) * stride] = __fmul_rn(x[u], product);
                }
        }
        piece_gates[((int64_t)blockIdx.x * heads + head) * dim + d] = product;
    }
}

// What a recurrence with a gate a channel reads, from a packed projection: q = act(projection) (act none or SiLU)
// and g = lower + (1 - lower) * sigmoid(projection + bias), a gate that never falls below `lower`; both float32
// [tokens, per].  `bias` and `lower` (float32 [per]) may be null: 0.
template <typename T>
__global__ void __launch_bounds__(256) gated_prepare_kernel(
    const T* __restrict__ proj, int64_t token_stride, int q_at, int g_at, int per, const float* __restrict__ bias,
    const float* __restrict__ lower, int q_act, float* __restrict__ q_out, float* __restrict__ g_out) {
    const int token = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    const T* row = proj + (int64_t)token * token_stride;
    const float x = to_float<T>(row[q_at + e]);
    q_out[(int64_t)token * per + e] = q_act ? __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))) : x;
    float z = to_float<T>(row[g_at + e]);
    if (bias) z = __fadd_rn(z, bias[e]);
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z)));
    const float low = lower ? lower[e] : 0.0f;
    g_out[(int64_t)token * per + e] = __fmaf_rn(__fsub_rn(1.0f, low), sig, low);
}

extern "C" int tvb_gated_prepare(const void* proj, long long token_stride, int q_at, int g_at, int per,
                                 const float* bias, const float* lower, int q_act, float* q_out, float* g_out,
                                 int tokens, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (per <= 0 || q_at < 0 || g_at < 0 || !q_out || !g_out) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    for (int first = 0; first < tokens; first += 65535) {
        const int count = min(65535, tokens - first);
        const dim3 grid((per + 255) / 256, count);
        if (dtype == TVB_F32)
            gated_prepare_kernel<float><<<grid, 256, 0, s>>>((const float*)proj + (int64_t)first * token_stride, token_stride,
                                                            q_at, g_at, per, bias, lower, q_act, q_out + (int64_t)first * per,
                                                            g_out + (int64_t)first * per);
        else if (dtype == TVB_BF16)
            gated_prepare_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)proj + (int64_t)first * token_stride, token_stride,
                                                           q_at, g_at, per, bias, lower, q_act, q_out + (int64_t)first * per,
                                                           g_out + (int64_t)first * per);
        else return TVB_BAD_ARGUMENT;
    }
    return tvb_last_error();
}

// One token a request (a decode step) of the recurrence with a gate a channel, the whole mixer between its two
// projections in one launch: a CTA a (request, head) reads the token's q, gate and v from the packed projection
// (q = act(q), g = lower + (1 - lower) sigmoid(g + bias), as gated_prepare), moves the head's state once,
// S <- diag(g) S + (1 - g) v^T, sums o = S^T q on the way, divides o by its root mean square (with `unit_norm`),
// multiplies by `norm_weight` and rounds once.  A thread owns VEC neighbouring columns of the state and one of
// SLICES slices of its rows; the slices' partial sums meet in shared memory in the order of the slices.
#define STEP_THREADS 256
template <typename T, int VEC>
__global__ void __launch_bounds__(STEP_THREADS) gated_step_kernel(
    const T* proj, int64_t token_stride, int q_at, int g_at, int v_at, const float* __restrict__ bias,
    const float* __restrict__ lower, int q_act, float* __restrict__ state, const int* __restrict__ row_starts,
    const int* __restrict__ state_slots, const int* __restrict__ token_row, const float* __restrict__ norm_weight,
    int unit_norm, float eps, T* __restrict__ out, int64_t out_stride, int heads, int dim, int vdim) {
    extern __shared__ __align__(16) float step_shared[];
    __shared__ float scratch[32];
    float* q_s = step_shared;                     // [dim]
    float* g_s = q_s + dim;                       // [dim]
    float* o_s = g_s + dim;                       // [slices][columns rounded up to VEC]
    const int row = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int token = row_starts[row];
    T* dst = out + (int64_t)token * out_stride + (int64_t)head * vdim;
    if (token_row[token] < 0) {                   // a padding row of a recorded batch: no request, no state
        for (int c = tid; c < vdim; c += STEP_THREADS) dst[c] = from_float<T>(0.0f);
        return;
    }
    const T* src = proj + (int64_t)token * token_stride;
    for (int d = tid; d < dim; d += STEP_THREADS) {
        const int e = head * dim + d;
        const float x = to_float<T>(src[q_at + e]);
        q_s[d] = q_act ? __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))) : x;
        float z = to_float<T>(src[g_at + e]);
        if (bias) z = __fadd_rn(z, bias[e]);
        const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z)));
        const float low = lower ? lower[e] : 0.0f;
        g_s[d] = __fmaf_rn(__fsub_rn(1.0f, low), sig, low);
    }
    __syncthreads();
    const int groups = (vdim + VEC - 1) / VEC;    // groups of VEC columns
    const int slices = max(1, STEP_THREADS / groups);
    const int group = tid % groups, slice = tid / groups;
    const int padded = groups * VEC;
    float* mine = state + (((int64_t)state_slots[row] * heads + head) * dim) * vdim;
    if (tid < groups * slices) {
        const int c = group * VEC;
        float vv[VEC], sum[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            vv[j] = c + j < vdim ? to_float<T>(src[v_at + head * vdim + c + j]) : 0.0f;
            sum[j] = 0.0f;
        }
        const int per = (dim + slices - 1) / slices;
        const int first = slice * per, last = min(dim, first + per);
        for (int d0 = first; d0 < last; d0 += 4) {            // four rows' loads are in flight together
            float s[4][VEC];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (d0 + u < last) {
                    const float* from = mine + (int64_t)(d0 + u) * vdim + c;
                    if constexpr (VEC == 4) {
                        const float4 x = *reinterpret_cast<const float4*>(from);
                        s[u][0] = x.x; s[u][1] = x.y; s[u][2] = x.z; s[u][3] = x.w;
                    } else s[u][0] = from[0];
                }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (d0 + u < last) {
                    const float g = g_s[d0 + u], k = __fsub_rn(1.0f, g), q = q_s[d0 + u];
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        s[u][j] = __fmaf_rn(k, vv[j], __fmul_rn(g, s[u][j]));
                        sum[j] = __fmaf_rn(s[u][j], q, sum[j]);
                    }
                    float* to = mine + (int64_t)(d0 + u) * vdim + c;
                    if constexpr (VEC == 4) *reinterpret_cast<float4*>(to) = make_float4(s[u][0], s[u][1], s[u][2], s[u][3]);
                    else to[0] = s[u][0];
                }
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) o_s[slice * padded + c + j] = sum[j];
    }
    __syncthreads();
    float part = 0.0f;
    for (int c = tid; c < vdim; c += STEP_THREADS) {
        float o = 0.0f;
        for (int sl = 0; sl < slices; ++sl) o = __fadd_rn(o, o_s[sl * padded + c]);
        o_s[c] = o;                                // slice 0's place: read by this thread alone before it is written
        part = __fmaf_rn(o, o, part);
    }
    float factor = 1.0f;
    if (unit_norm) {
        const float squares = block_sum(part, scratch);
        factor = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, (float)vdim), eps)));
    }
    for (int c = tid; c < vdim; c += STEP_THREADS) {
        float x = __fmul_rn(o_s[c], factor);
        if (norm_weight) x = __fmul_rn(x, norm_weight[c]);
        dst[c] = from_float<T>(x);
    }
}

// proj [rows of one token each, columns] of the storage type; state float32 [slots, heads, dim, vdim]; every entry
// of row_starts [rows + 1] holds one token; out [tokens, heads * vdim] of the storage type.
extern "C" int tvb_gated_step(const void* proj, long long token_stride, int q_at, int g_at, int v_at, const float* bias,
                              const float* lower, int q_act, float* state, const int* row_starts,
                              const int* state_slots, const int* token_row, const float* norm_weight, int unit_norm,
                              float eps, void* out, long long out_stride, int rows, int heads, int dim, int vdim,
                              int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || dim <= 0 || dim > 256 || vdim <= 0 || vdim > 4 * STEP_THREADS || !state)
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const bool by_four = vdim % 4 == 0 && ((uintptr_t)state & 15) == 0;
    const int vec = by_four ? 4 : 1;
    if (!by_four && vdim > STEP_THREADS) return TVB_BAD_ARGUMENT;
    const int groups = (vdim + vec - 1) / vec, slices = STEP_THREADS / groups > 0 ? STEP_THREADS / groups : 1;
    const size_t smem = (size_t)(2 * dim + slices * groups * vec) * sizeof(float);
    const dim3 grid(rows, heads);
#define GO(T, V) gated_step_kernel<T, V><<<grid, STEP_THREADS, smem, s>>>(                                          \
        (const T*)proj, token_stride, q_at, g_at, v_at, bias, lower, q_act, state, row_starts, state_slots, token_row, \
        norm_weight, unit_norm, eps, (T*)out, out_stride, heads, dim, vdim)
    if (dtype == TVB_F32) { if (by_four) GO(float, 4); else GO(float, 1); }
    else if (dtype == TVB_BF16) { if (by_four) GO(bf16, 4); else GO(bf16, 1); }
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}

#define RET_ACT_NONE 0
#define RET_ACT_SILU 1
#define RET_ACT_SIGMOID 2

// A warp a (token, head): o / sqrt(mean(o^2) + eps) (with `unit_norm`; times `norm_weight` [vdim], one for all
// heads, if given), times act(gate).
template <typename T>
__global__ void __launch_bounds__(128) retention_finish_kernel(
    const float* __restrict__ o, const T* gate, int64_t gate_stride, T* __restrict__ out, int64_t out_stride,
    int tokens, int heads, int vdim, int unit_norm, float eps, int act, const float* __restrict__ norm_weight) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + warp;
    if (item >= (int64_t)tokens * heads) return;
    const int token = (int)(item / heads), head = (int)(item % heads);
    const float* src = o + ((int64_t)token * heads + head) * vdim;
    float factor = 1.0f;
    if (unit_norm) {
        float squares = 0.0f;
        for (int i = lane; i < vdim; i += 32) squares = __fmaf_rn(src[i], src[i], squares);
        squares = warp_sum(squares);
        factor = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, (float)vdim), eps)));
    }
    const T* g = gate ? gate + (int64_t)token * gate_stride + (int64_t)head * vdim : nullptr;
    T* dst = out + (int64_t)token * out_stride + (int64_t)head * vdim;
    for (int i = lane; i < vdim; i += 32) {
        float x = __fmul_rn(src[i], factor);
        if (norm_weight) x = __fmul_rn(x, norm_weight[i]);
        if (g) {
            const float z = to_float<T>(g[i]);
            const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z)));
            x = __fmul_rn(x, act == RET_ACT_SILU ? __fmul_rn(z, sig) : act == RET_ACT_SIGMOID ? sig : z);
        }
        dst[i] = from_float<T>(x);
    }
}

extern "C" int tvb_retention_prepare(const void* proj, long long token_stride, int q_at, int k_at, int heads, int dim,
                                     const float* inv_freq, int rot_dims, int pairing, float key_scale,
                                     const int* positions, float* q_out, float* k_out, int tokens, int dtype,
                                     void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || dim <= 0 || (inv_freq && (rot_dims <= 0 || rot_dims % 2 || rot_dims > dim ||
                                                rot_dims / 2 > RET_MAX_TURNED || pairing < 0 || pairing > 1)))
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    // few tokens: slices of a row's 2 * heads * dim elements go to CTAs of their own, up to eight elements a thread
    const int slices = tokens >= 1024 ? 1 : max(1, min(64, (2 * heads * dim + 1023) / 1024));
    const dim3 tokens_by_slices(tokens, slices);
    if (dtype == TVB_F32)
        retention_prepare_kernel<float><<<tokens_by_slices, 128, 0, s>>>((const float*)proj, token_stride, q_at, k_at, heads, dim,
                                                               inv_freq, rot_dims, pairing, key_scale, positions, q_out, k_out);
    else if (dtype == TVB_BF16)
        retention_prepare_kernel<bf16><<<tokens_by_slices, 128, 0, s>>>((const bf16*)proj, token_stride, q_at, k_at, heads, dim,
                                                              inv_freq, rot_dims, pairing, key_scale, positions, q_out, k_out);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}

extern "C" int tvb_retention_max_dim() { return 256; }

// q, k: float32 [tokens, heads * dim]; v: [tokens, >= heads * vdim] of the storage type with rows
// `v_stride` elements apart; state: float32 [slots, heads, dim, vdim]; decay: float32 [heads];
// row_starts [rows + 1], state_slots [rows], token_row [tokens] (negative: padding); out: float32
// [tokens, heads * vdim].  `lanes` (0: the fewest, or more where a B200's 148 SMs would idle) is the number of lanes that share a tile of eight columns
// of the state: 4, 8, 16 or 32, with at most eight rows of the key a lane (lanes * 8 >= dim).
//
// segment == 0: a CTA walks a whole entry, from the request's state to the state it leaves.
// segment > 0: every entry is cut into pieces of `segment` tokens that run side by side (three launches):
// each piece from a state of zero, which leaves o without what came before the piece and, in
// parts [pieces, heads, dim, vdim], what the piece adds; then the states the pieces start from, along every
// entry; then decay^(t + 1) S_start^T q_t added to the piece's token t.  `pieces` is at least the number of
// pieces of all entries (tokens / segment + rows always is).
//
// A library compiled with RET_GATED takes `gates` (float32 [tokens, heads * dim]) instead of `decay`, and with
// RET_GATED == 1 no `k`; in pieces it also wants `scaled_q` (float32, the size of q) and `piece_gates` (float32
// [pieces, heads, dim]) as scratch.
extern "C" int tvb_retention_scan(const float* q, const float* k, const void* v, long long v_stride, float* state,
                                  const float* decay, const int* row_starts, const int* state_slots,
                                  const int* token_row, float* out, int rows, int heads, int dim, int vdim,
                                  int lanes, float* parts, int segment, int pieces, int dtype,
                                  const float* gates, float* scaled_q, float* piece_gates, void* stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || dim <= 0 || dim > 256 || vdim <= 0 || rows > 65535 || segment < 0 ||
        (segment > 0 && (!parts || pieces <= 0)))
        return TVB_BAD_ARGUMENT;
#if RET_GATED
    if (!gates || (RET_GATED == 2 && !k) || (segment > 0 && (!scaled_q || !piece_gates))) return TVB_BAD_ARGUMENT;
#else
    if (!decay || !k || gates) return TVB_BAD_ARGUMENT;
#endif
    const int blocks = segment > 0 ? pieces : rows;
    if (lanes == 0) {                             // the fewest that hold the key, more while SMs would idle
        for (lanes = 4; lanes < 32 && lanes * 8 < dim; lanes *= 2) {}
        while (lanes < 32 && (long long)blocks * heads * ((vdim + RET_THREADS / lanes * RET_TILE - 1) /
                                                          (RET_THREADS / lanes * RET_TILE)) < 2 * 148)
            lanes *= 2;
    }
    if ((lanes != 4 && lanes != 8 && lanes != 16 && lanes != 32) || lanes * 8 < dim) return TVB_BAD_ARGUMENT;
    const int cols = RET_THREADS / lanes * RET_TILE;
    const dim3 grid(blocks, heads, (vdim + cols - 1) / cols);
    if (grid.z > 65535) return TVB_BAD_ARGUMENT;
    const bool few = (dim + lanes - 1) / lanes <= 4;          // rows of the state a lane: four or eight
    cudaStream_t s = (cudaStream_t)stream;
#define GO(T, G, R, C) retention_scan_kernel<T, G, R, C><<<grid, RET_THREADS, 0, s>>>(                              \
        (C && RET_GATED) ? scaled_q : q, k, gates, (const T*)v, v_stride, state, decay, row_starts, state_slots,   \
        token_row, out, parts, segment, rows, heads, dim, vdim)
#define BY_ROWS(T, G, C)                                                                                           \
    if (few) GO(T, G, 4, C);                                                                                       \
    else GO(T, G, 8, C)
#define BY_LANES(T, C)                                                                                             \
    if (lanes == 4) { BY_ROWS(T, 4, C); }                                                                          \
    else if (lanes == 8) { BY_ROWS(T, 8, C); }                                                                     \
    else if (lanes == 16) { BY_ROWS(T, 16, C); }                                                                   \
    else { BY_ROWS(T, 32, C); }
    if (dtype == TVB_F32) { BY_LANES(float, false) }
    else if (dtype == TVB_BF16) { BY_LANES(bf16, false) }
    else return TVB_BAD_ARGUMENT;
    if (segment > 0) {
        const int per = dim * vdim;
#if RET_GATED
        retention_gate_prefix_kernel<<<dim3(pieces, heads), 128, 0, s>>>(q, gates, scaled_q, piece_gates, row_starts,
                                                                        token_row, segment, rows, heads, dim);
#endif
        // four elements a thread where they lie in one row of the state (gates: one decay for the four)
        if ((RET_GATED ? vdim : per) % 4 == 0 && (((uintptr_t)state | (uintptr_t)parts) & 15) == 0)
            retention_combine_kernel<4><<<dim3((per / 4 + 255) / 256, heads, rows), 256, 0, s>>>(
                state, parts, decay, piece_gates, row_starts, state_slots, token_row, segment, heads, per, vdim);
        else
            retention_combine_kernel<1><<<dim3((per + 255) / 256, heads, rows), 256, 0, s>>>(
                state, parts, decay, piece_gates, row_starts, state_slots, token_row, segment, heads, per, vdim);
        BY_LANES(float, true)                     // the correcting pass reads no values: one type will do
    }
#undef BY_LANES
#undef BY_ROWS
#undef GO
    return tvb_last_error();
}

// o: float32 [tokens, heads * vdim]; gate (or null) and out of the storage type, rows may be strided.
extern "C" int tvb_retention_finish(const float* o, const void* gate, long long gate_stride, void* out,
                                    long long out_stride, int tokens, int heads, int vdim, int unit_norm, float eps,
                                    int act, const float* norm_weight, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || act < 0 || act > 2) return TVB_BAD_ARGUMENT;
    const long long blocks = ((long long)tokens * heads + 3) / 4;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TVB_F32)
        retention_finish_kernel<float><<<(unsigned)blocks, 128, 0, s>>>(o, (const float*)gate, gate_stride, (float*)out,
                                                                        out_stride, tokens, heads, vdim, unit_norm, eps, act, norm_weight);
    else if (dtype == TVB_BF16)
        retention_finish_kernel<bf16><<<(unsigned)blocks, 128, 0, s>>>(o, (const bf16*)gate, gate_stride, (bf16*)out,
                                                                       out_stride, tokens, heads, vdim, unit_norm, eps, act, norm_weight);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}
