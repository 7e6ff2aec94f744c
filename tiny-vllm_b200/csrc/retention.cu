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
//                       from; a CTA has one (request, head, 32 value columns), a thread a quarter of
//                       one column of the state in registers; tokens come in blocks of eight through
//                       shared memory, the next block's loads in flight while this one is computed
//   retention_finish    every head's o divided by its root mean square (or not), times act(gate),
//                       rounded once to the storage type
//
// Angles, the rotated q and k, the outer products, the state and the sums are float32 whatever the
// storage type; only v and the gate are read in it and only the finished output is rounded to it.
#include "common.cuh"

#define RET_PAIR_INTERLEAVED 0
#define RET_PAIR_HALF_SPLIT 1
#define RET_MAX_TURNED 512        // pairs of a head that turn: sine and cosine of a token in shared memory

template <typename T>
__global__ void __launch_bounds__(128) retention_prepare_kernel(
    const T* __restrict__ proj, int64_t token_stride, int q_at, int k_at, int heads, int dim,
    const float* __restrict__ inv_freq, int rot_dims, int pairing, float key_scale,
    const int* __restrict__ positions, float* __restrict__ q_out, float* __restrict__ k_out) {
    __shared__ float cos_s[RET_MAX_TURNED], sin_s[RET_MAX_TURNED];
    const int token = blockIdx.x;
    const int half = inv_freq ? rot_dims >> 1 : 0;
    const float position = (float)max(positions[token], 0);
    for (int j = threadIdx.x; j < half; j += blockDim.x)
        sincosf(__fmul_rn(position, inv_freq[j]), &sin_s[j], &cos_s[j]);
    __syncthreads();
    const T* row = proj + (int64_t)token * token_stride;
    const int per = heads * dim;
    for (int e = threadIdx.x; e < 2 * per; e += blockDim.x) {
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
#define RET_GROUPS 4                              // threads that share a column of the state
#define RET_COLS (RET_THREADS / RET_GROUPS)       // value columns a CTA
#define RET_BLOCK 8                               // tokens that wait in shared memory

// ROWS: rows of the state a thread holds (dim <= RET_GROUPS * ROWS)
template <typename T, int ROWS>
__global__ void __launch_bounds__(RET_THREADS) retention_scan_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const T* __restrict__ v, int64_t v_stride,
    float* __restrict__ state, const float* __restrict__ decay, const int* __restrict__ row_starts,
    const int* __restrict__ state_slots, const int* __restrict__ token_row, float* __restrict__ out,
    int heads, int dim, int vdim) {
    constexpr int LOADS = RET_BLOCK * RET_GROUPS * ROWS / RET_THREADS;      // q (and k) values a thread fetches a block
    __shared__ float q_s[RET_BLOCK][RET_GROUPS * ROWS];
    __shared__ float k_s[RET_BLOCK][RET_GROUPS * ROWS];
    __shared__ float v_s[RET_BLOCK][RET_COLS];
    const int row = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * RET_COLS;
    const int tid = threadIdx.x, group = tid % RET_GROUPS, col = tid / RET_GROUPS;
    const int begin = row_starts[row], count = row_starts[row + 1] - begin;
    if (count <= 0) return;
    const int c = col0 + col;
    const bool live = c < vdim;
    if (token_row[begin] < 0) {                   // a padding row of a recorded batch: no request, no state
        if (live && group == 0)
            for (int t = 0; t < count; ++t) out[(int64_t)(begin + t) * heads * vdim + (int64_t)head * vdim + c] = 0.0f;
        return;
    }
    const float a = decay[head];
    float* mine = state + (((int64_t)state_slots[row] * heads + head) * dim) * vdim + c;
    float s[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int d = group + RET_GROUPS * i;
        s[i] = (live && d < dim) ? mine[(int64_t)d * vdim] : 0.0f;
    }
    const int64_t qk_stride = (int64_t)heads * dim;
    const float* q_head = q + (int64_t)begin * qk_stride + (int64_t)head * dim;
    const float* k_head = k + (int64_t)begin * qk_stride + (int64_t)head * dim;
    const T* v_head = v + (int64_t)begin * v_stride + (int64_t)head * vdim + col0;
    const int width = RET_GROUPS * ROWS;
    float q_next[LOADS], k_next[LOADS], v_next[2];

    auto fetch = [&](int first) {                 // tokens first .. first + RET_BLOCK - 1 into registers
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int e = tid + RET_THREADS * j, t = e / width, d = e % width;
            const bool ok = first + t < count && d < dim;
            q_next[j] = ok ? q_head[(int64_t)(first + t) * qk_stride + d] : 0.0f;
            k_next[j] = ok ? k_head[(int64_t)(first + t) * qk_stride + d] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int e = tid + RET_THREADS * j, t = e / RET_COLS, cc = e % RET_COLS;
            const bool ok = first + t < count && col0 + cc < vdim;
            v_next[j] = ok ? to_float<T>(v_head[(int64_t)(first + t) * v_stride + cc]) : 0.0f;
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int e = tid + RET_THREADS * j;
            q_s[e / width][e % width] = q_next[j];
            k_s[e / width][e % width] = k_next[j];
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int e = tid + RET_THREADS * j;
            v_s[e / RET_COLS][e % RET_COLS] = v_next[j];
        }
    };

    fetch(0);
    for (int first = 0; first < count; first += RET_BLOCK) {
        __syncthreads();                          // the block before is read
        stage();
        __syncthreads();
        if (first + RET_BLOCK < count) fetch(first + RET_BLOCK);
        const int here = min(RET_BLOCK, count - first);
        for (int t = 0; t < here; ++t) {
            const float vt = v_s[t][col];
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int d = group + RET_GROUPS * i;
                s[i] = __fmaf_rn(k_s[t][d], vt, __fmul_rn(a, s[i]));
                sum = __fmaf_rn(s[i], q_s[t][d], sum);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (live && group == 0)
                out[(int64_t)(begin + first + t) * heads * vdim + (int64_t)head * vdim + c] = sum;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int d = group + RET_GROUPS * i;
            if (d < dim) mine[(int64_t)d * vdim] = s[i];
        }
    }
}

#define RET_ACT_NONE 0
#define RET_ACT_SILU 1
#define RET_ACT_SIGMOID 2

// A warp a (token, head): o / sqrt(mean(o^2) + eps) (with `unit_norm`), times act(gate).
template <typename T>
__global__ void __launch_bounds__(128) retention_finish_kernel(
    const float* __restrict__ o, const T* gate, int64_t gate_stride, T* __restrict__ out, int64_t out_stride,
    int tokens, int heads, int vdim, int unit_norm, float eps, int act) {
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
    if (dtype == TVB_F32)
        retention_prepare_kernel<float><<<tokens, 128, 0, s>>>((const float*)proj, token_stride, q_at, k_at, heads, dim,
                                                               inv_freq, rot_dims, pairing, key_scale, positions, q_out, k_out);
    else if (dtype == TVB_BF16)
        retention_prepare_kernel<bf16><<<tokens, 128, 0, s>>>((const bf16*)proj, token_stride, q_at, k_at, heads, dim,
                                                              inv_freq, rot_dims, pairing, key_scale, positions, q_out, k_out);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}

extern "C" int tvb_retention_max_dim() { return RET_GROUPS * 64; }

// q, k: float32 [tokens, heads * dim]; v: [tokens, >= heads * vdim] of the storage type with rows
// `v_stride` elements apart; state: float32 [slots, heads, dim, vdim]; decay: float32 [heads];
// row_starts [rows + 1], state_slots [rows], token_row [tokens] (negative: padding); out: float32
// [tokens, heads * vdim].
extern "C" int tvb_retention_scan(const float* q, const float* k, const void* v, long long v_stride, float* state,
                                  const float* decay, const int* row_starts, const int* state_slots,
                                  const int* token_row, float* out, int rows, int heads, int dim, int vdim,
                                  int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || dim <= 0 || dim > RET_GROUPS * 64 || vdim <= 0) return TVB_BAD_ARGUMENT;
    const dim3 grid(rows, heads, (vdim + RET_COLS - 1) / RET_COLS);
    if (grid.z > 65535) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
#define GO(T, ROWS) retention_scan_kernel<T, ROWS><<<grid, RET_THREADS, 0, s>>>(                                   \
        q, k, (const T*)v, v_stride, state, decay, row_starts, state_slots, token_row, out, heads, dim, vdim)
#define BY_DIM(T)                                                                                                  \
    if (dim <= RET_GROUPS * 8) GO(T, 8);                                                                           \
    else if (dim <= RET_GROUPS * 16) GO(T, 16);                                                                    \
    else if (dim <= RET_GROUPS * 32) GO(T, 32);                                                                    \
    else GO(T, 64)
    if (dtype == TVB_F32) { BY_DIM(float); }
    else if (dtype == TVB_BF16) { BY_DIM(bf16); }
    else return TVB_BAD_ARGUMENT;
#undef BY_DIM
#undef GO
    return tvb_last_error();
}

// o: float32 [tokens, heads * vdim]; gate (or null) and out of the storage type, rows may be strided.
extern "C" int tvb_retention_finish(const float* o, const void* gate, long long gate_stride, void* out,
                                    long long out_stride, int tokens, int heads, int vdim, int unit_norm, float eps,
                                    int act, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || act < 0 || act > 2) return TVB_BAD_ARGUMENT;
    const long long blocks = ((long long)tokens * heads + 3) / 4;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TVB_F32)
        retention_finish_kernel<float><<<(unsigned)blocks, 128, 0, s>>>(o, (const float*)gate, gate_stride, (float*)out,
                                                                        out_stride, tokens, heads, vdim, unit_norm, eps, act);
    else if (dtype == TVB_BF16)
        retention_finish_kernel<bf16><<<(unsigned)blocks, 128, 0, s>>>(o, (const bf16*)gate, gate_stride, (bf16*)out,
                                                                       out_stride, tokens, heads, vdim, unit_norm, eps, act);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}
