// From a packed projection row to prepared queries and cached keys and values, for attention
// mixers whose sizes and steps are all parameters.  A block per token, a warp per head.
//
//   q heads   [optional RMS norm over the head, with or without a weight] -> [optional rotation]
//             -> written back where they stand
//   k heads   the same, then written to the key cache at the token's slot
//   v heads   [optional blend (1 - l) v + l v_first with a scalar l read from the device]
//             -> written to the value cache
//
// With biases (float32: one number a column of the q heads, the k heads and the v heads) the projection
// is taken as proj + bias, before anything else.  The v heads may be read from the k columns
// (v_at == k_at): k is never changed where it stands.
//
// Keys are `key_dim` wide, values `value_dim`; the caches are [pages, num_kv, page, dim].
// Rotation: the first `rot_dims` dimensions of a head turn by position * inv_freq[i]; pair i is
// (2i, 2i + 1) with the interleaved pairing and (i, i + rot_dims / 2) with the half-split one;
// the rest passes unchanged.  Angles are float32 products of the position and the frequency,
// sine and cosine are the accurate ones.  Norm, rotation and blend are float32 with one
// rounding, when the value is stored.
#include "common.cuh"

#define PREP_MAX_PAIRS 4      // pairs per lane: heads of up to 256
#define PREP_NORM_NONE 0
#define PREP_NORM_UNIT 1
#define PREP_NORM_WEIGHT 2
#define PREP_PAIR_INTERLEAVED 0
#define PREP_PAIR_HALF_SPLIT 1

// two neighbouring values of the storage type in one access where the address allows it
template <typename T> __device__ __forceinline__ void load_pair(const T* p, float& a, float& b) {
    a = to_float<T>(p[0]);
    b = to_float<T>(p[1]);
}
template <> __device__ __forceinline__ void load_pair<bf16>(const bf16* p, float& a, float& b) {
    if (((uintptr_t)p & 3) == 0) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        a = v.x;
        b = v.y;
    } else {
        a = __bfloat162float(p[0]);
        b = __bfloat162float(p[1]);
    }
}
template <typename T> __device__ __forceinline__ void store_pair(T* p, float a, float b) {
    p[0] = from_float<T>(a);
    p[1] = from_float<T>(b);
}
template <> __device__ __forceinline__ void store_pair<bf16>(bf16* p, float a, float b) {
    if (((uintptr_t)p & 3) == 0) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    else { p[0] = __float2bfloat16_rn(a); p[1] = __float2bfloat16_rn(b); }
}

// A block of PREP_WARPS warps takes PREP_WARPS consecutive heads of one token (grid: tokens x groups of
// heads): sine and cosine of the token's angles are taken once a block, into shared memory, then
// every warp has one head (a q head, a k head or a v head).  Few heads a block keep the chains of
// dependent loads short: a decode step has only a handful of tokens to spread over the GPU.
#define PREP_WARPS 4

// PAIRS: pairs of a head a lane holds (heads of up to 64 * PAIRS)
template <typename T, typename W, int PAIRS>
__global__ void __launch_bounds__(PREP_WARPS * 32) qkv_prepare_kernel(
    T* proj, int64_t token_stride, int q_at, int k_at, int v_at, int num_q, int num_kv, int key_dim,
    int value_dim, int norm_mode, const W* __restrict__ q_weight, const W* __restrict__ k_weight, float eps,
    const float* __restrict__ inv_freq, int rot_dims, int pairing, const int* __restrict__ positions,
    const int* __restrict__ slots, T* __restrict__ key_cache, T* __restrict__ value_cache, int page_size,
    const T* v_first, int64_t v_first_stride, const T* __restrict__ blend, int tokens,
    const float* __restrict__ q_bias, const float* __restrict__ k_bias, const float* __restrict__ v_bias) {
    __shared__ float cos_s[32 * PAIRS], sin_s[32 * PAIRS];
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = num_q + 2 * num_kv;
    T* token_row = proj + (int64_t)token * token_stride;
    const int slot = slots ? slots[token] : -1;
    const int pairs = key_dim >> 1, turned = inv_freq ? rot_dims >> 1 : 0;
    const float position = (float)max(positions[token], 0);
    const int first_head = blockIdx.y * PREP_WARPS;
    if (first_head < num_q + num_kv) {                      // a block of value heads alone turns nothing
        for (int j = threadIdx.x; j < turned; j += blockDim.x)
            sincosf(__fmul_rn(position, inv_freq[j]), &sin_s[j], &cos_s[j]);
    }
    __syncthreads();

    for (int head = first_head + warp; head < min(heads, first_head + PREP_WARPS); head += PREP_WARPS) {
        if (head >= num_q + num_kv) {                       // a value head
            if (slot < 0) continue;
            const int g = head - num_q - num_kv;
            const T* src = token_row + v_at + (int64_t)g * value_dim;
            T* dst = value_cache + (((int64_t)(slot / page_size) * num_kv + g) * page_size + slot % page_size) * value_dim;
            const float* vb = v_bias ? v_bias + (int64_t)g * value_dim : nullptr;
            if (vb && !v_first) {
                for (int i = lane; i < value_dim; i += 32) dst[i] = from_float<T>(__fadd_rn(to_float<T>(src[i]), vb[i]));
            } else if (v_first) {
                const float l = to_float<T>(blend[0]);
                const float keep = __fsub_rn(1.0f, l);
                const T* first = v_first + (int64_t)token * v_first_stride + (int64_t)g * value_dim;
                for (int i = 2 * lane; i + 1 < value_dim; i += 64) {
                    float a, b, fa, fb;
                    load_pair<T>(src + i, a, b);
                    load_pair<T>(first + i, fa, fb);
                    store_pair<T>(dst + i, __fadd_rn(__fmul_rn(keep, a), __fmul_rn(l, fa)),
                                  __fadd_rn(__fmul_rn(keep, b), __fmul_rn(l, fb)));
                }
                if ((value_dim & 1) && lane == 0) {
                    const int i = value_dim - 1;
                    dst[i] = from_float<T>(__fadd_rn(__fmul_rn(keep, to_float<T>(src[i])),
                                                     __fmul_rn(l, to_float<T>(first[i]))));
                }
            } else {
                for (int i = 2 * lane; i + 1 < value_dim; i += 64) {
                    float a, b;
                    load_pair<T>(src + i, a, b);          // widening and rounding back changes no bit
                    store_pair<T>(dst + i, a, b);
                }
                if ((value_dim & 1) && lane == 0) dst[value_dim - 1] = src[value_dim - 1];
            }
            continue;
        }
        const bool is_key = head >= num_q;
        if (is_key && slot < 0) continue;
        T* src = is_key ? token_row + k_at + (int64_t)(head - num_q) * key_dim : token_row + q_at + (int64_t)head * key_dim;
        T* dst = is_key ? key_cache + (((int64_t)(slot / page_size) * num_kv + (head - num_q)) * page_size +
                                       slot % page_size) * key_dim
                        : src;
        const W* weight = norm_mode == PREP_NORM_WEIGHT ? (is_key ? k_weight : q_weight) : nullptr;
        const float* added = is_key ? (k_bias ? k_bias + (int64_t)(head - num_q) * key_dim : nullptr)
                                    : (q_bias ? q_bias + (int64_t)head * key_dim : nullptr);

        // pair j of the head: the two dimensions it holds
        int at_a[PAIRS], at_b[PAIRS];
        float a[PAIRS], b[PAIRS];
        float squares = 0.0f;
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
            const int j = lane + 32 * i;
            a[i] = b[i] = 0.0f;
            at_a[i] = at_b[i] = 0;
            if (j < pairs) {
                if (pairing == PREP_PAIR_HALF_SPLIT && j < turned) {
                    at_a[i] = j; at_b[i] = j + turned;
                    a[i] = to_float<T>(src[at_a[i]]);
                    b[i] = to_float<T>(src[at_b[i]]);
                } else {
                    at_a[i] = 2 * j; at_b[i] = 2 * j + 1;
                    load_pair<T>(src + 2 * j, a[i], b[i]);
                }
                if (added) { a[i] = __fadd_rn(a[i], added[at_a[i]]); b[i] = __fadd_rn(b[i], added[at_b[i]]); }
                squares = __fadd_rn(squares, __fmaf_rn(a[i], a[i], __fmul_rn(b[i], b[i])));
            }
        }
        // a head of an odd size has one value without a partner (never turned): lane 0 carries it
        const bool lone_here = (key_dim & 1) && lane == 0;
        float lone = lone_here ? to_float<T>(src[key_dim - 1]) : 0.0f;
        if (lone_here && added) lone = __fadd_rn(lone, added[key_dim - 1]);
        squares = __fmaf_rn(lone, lone, squares);
        if (norm_mode != PREP_NORM_NONE) {
            squares = warp_sum(squares);
            const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, (float)key_dim), eps)));
            lone = __fmul_rn(lone, inverse_rms);
            if (weight && lone_here) lone = __fmul_rn(lone, to_float<W>(weight[key_dim - 1]));
#pragma unroll
            for (int i = 0; i < PAIRS; ++i) {
                if (lane + 32 * i < pairs) {
                    a[i] = __fmul_rn(a[i], inverse_rms);
                    b[i] = __fmul_rn(b[i], inverse_rms);
                    if (weight) {
                        a[i] = __fmul_rn(a[i], to_float<W>(weight[at_a[i]]));
                        b[i] = __fmul_rn(b[i], to_float<W>(weight[at_b[i]]));
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < PAIRS; ++i) {
            const int j = lane + 32 * i;
            if (j < pairs) {
                float u = a[i], v = b[i];
                if (j < turned) {
                    const float s = sin_s[j], c = cos_s[j];
                    u = __fsub_rn(__fmul_rn(a[i], c), __fmul_rn(b[i], s));
                    v = __fadd_rn(__fmul_rn(b[i], c), __fmul_rn(a[i], s));
                }
                if (at_b[i] == at_a[i] + 1) store_pair<T>(dst + at_a[i], u, v);
                else { dst[at_a[i]] = from_float<T>(u); dst[at_b[i]] = from_float<T>(v); }
            }
        }
        if (lone_here) dst[key_dim - 1] = from_float<T>(lone);
    }
}

// bfloat16, heads of 16, 32, 64, 128 or 256 keys, every offset a multiple of 8, neighbouring pairs
// (or no rotation): a block per token; a lane holds eight consecutive values of a head (four
// pairs) in one 16-byte word, the key_dim / 8 lanes of a head sit side by side in a warp and sum
// their squares with shuffles; sine and cosine are taken once a token.  An eighth of the
// instructions of the general kernel for the same bytes.
template <typename W>
__global__ void __launch_bounds__(PREP_WARPS * 32) qkv_prepare_wide_kernel(
    bf16* proj, int64_t token_stride, int q_at, int k_at, int v_at, int num_q, int num_kv, int key_dim,
    int value_dim, int norm_mode, const W* __restrict__ q_weight, const W* __restrict__ k_weight, float eps,
    const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
    const int* __restrict__ slots, bf16* __restrict__ key_cache, bf16* __restrict__ value_cache, int page_size,
    const bf16* v_first, int64_t v_first_stride, const bf16* __restrict__ blend,
    const float* __restrict__ q_bias, const float* __restrict__ k_bias, const float* __restrict__ v_bias) {
    __shared__ float cos_s[32 * PREP_MAX_PAIRS], sin_s[32 * PREP_MAX_PAIRS];
    const int token = blockIdx.x, tid = threadIdx.x;
    const int lanes = key_dim >> 3;                        // lanes a head: 2, 4, 8, 16 or 32
    const int turned = inv_freq ? rot_dims >> 1 : 0;
    const float position = (float)max(positions[token], 0);
    for (int j = tid; j < turned; j += blockDim.x) sincosf(__fmul_rn(position, inv_freq[j]), &sin_s[j], &cos_s[j]);
    __syncthreads();
    bf16* token_row = proj + (int64_t)token * token_stride;
    const int slot = slots ? slots[token] : -1;
    const int64_t page_row = slot >= 0 ? (int64_t)(slot / page_size) * num_kv : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;
    const int items = (num_q + num_kv) * lanes;
    for (int first = 0; first < items; first += blockDim.x) {
        const int item = first + tid;
        const bool live = item < items;
        const int head = live ? item / lanes : 0, c = live ? item % lanes : 0;
        const bool is_key = head >= num_q;
        bf16* src = token_row + (is_key ? k_at + (int64_t)(head - num_q) * key_dim : q_at + (int64_t)head * key_dim) + c * 8;
        float x[8];
        if (live) {
            unpack_bf16x8(ld_global_16(src), x);
            const float* added = is_key ? (k_bias ? k_bias + (int64_t)(head - num_q) * key_dim + c * 8 : nullptr)
                                        : (q_bias ? q_bias + (int64_t)head * key_dim + c * 8 : nullptr);
            if (added) {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = __fadd_rn(x[i], added[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = 0.0f;
        }
        if (norm_mode != PREP_NORM_NONE) {
            float squares = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) squares = __fmaf_rn(x[i], x[i], squares);
            for (int delta = lanes >> 1; delta > 0; delta >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, delta);
            const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, (float)key_dim), eps)));
            const W* weight = norm_mode == PREP_NORM_WEIGHT ? (is_key ? k_weight : q_weight) + c * 8 : nullptr;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x[i] = __fmul_rn(x[i], inverse_rms);
                if (weight) x[i] = __fmul_rn(x[i], to_float<W>(weight[i]));
            }
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int j = c * 4 + p;
            if (j < turned) {
                const float s = sin_s[j], co = cos_s[j], u = x[2 * p], v = x[2 * p + 1];
                x[2 * p] = __fsub_rn(__fmul_rn(u, co), __fmul_rn(v, s));
                x[2 * p + 1] = __fadd_rn(__fmul_rn(v, co), __fmul_rn(u, s));
            }
        }
        if (!live) continue;
        if (!is_key) *reinterpret_cast<uint4*>(src) = pack_bf16x8(x);
        else if (slot >= 0)
            *reinterpret_cast<uint4*>(key_cache + ((page_row + (head - num_q)) * page_size + in_page) * key_dim + c * 8) =
                pack_bf16x8(x);
    }
    if (slot < 0) return;
    const int per_head = value_dim >> 3;
    const float l = v_first ? __bfloat162float(blend[0]) : 0.0f, keep = __fsub_rn(1.0f, l);
    for (int item = tid; item < num_kv * per_head; item += blockDim.x) {
        const int g = item / per_head, c = item % per_head;
        uint4 word = ld_global_16(token_row + v_at + (int64_t)g * value_dim + c * 8);
        if (v_bias) {
            float x[8];
            unpack_bf16x8(word, x);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fadd_rn(x[i], v_bias[(int64_t)g * value_dim + c * 8 + i]);
            word = pack_bf16x8(x);
        }
        if (v_first) {
            float x[8], f[8];
            unpack_bf16x8(word, x);
            unpack_bf16x8(ld_global_16(v_first + (int64_t)token * v_first_stride + (int64_t)g * value_dim + c * 8), f);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __fadd_rn(__fmul_rn(keep, x[i]), __fmul_rn(l, f[i]));
            word = pack_bf16x8(x);
        }
        *reinterpret_cast<uint4*>(value_cache + ((page_row + g) * page_size + in_page) * value_dim + c * 8) = word;
    }
}

template <typename T, typename W>
static int launch_prepare(void* proj, long long token_stride, int q_at, int k_at, int v_at, int num_q, int num_kv,
                          int key_dim, int value_dim, int norm_mode, const void* qw, const void* kw, float eps,
                          const float* inv_freq, int rot_dims, int pairing, const int* positions, const int* slots,
                          void* key_cache, void* value_cache, int page_size, const void* v_first,
                          long long v_first_stride, const void* blend, int tokens, const float* q_bias,
                          const float* k_bias, const float* v_bias, cudaStream_t s) {
    const int heads = num_q + 2 * num_kv;
    const dim3 grid((unsigned)tokens, (unsigned)((heads + PREP_WARPS - 1) / PREP_WARPS));
#define GO(PAIRS)                                                                                                   \
    qkv_prepare_kernel<T, W, PAIRS><<<grid, PREP_WARPS * 32, 0, s>>>(                                               \
        (T*)proj, token_stride, q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim, norm_mode, (const W*)qw,       \
        (const W*)kw, eps, inv_freq, rot_dims, pairing, positions, slots, (T*)key_cache, (T*)value_cache,           \
        page_size, (const T*)v_first, v_first_stride, (const T*)blend, tokens, q_bias, k_bias, v_bias)
    if (key_dim <= 64) GO(1);
    else if (key_dim <= 128) GO(2);
    else GO(PREP_MAX_PAIRS);
#undef GO
    return tvb_last_error();
}

extern "C" int tvb_qkv_prepare_biased(void* proj, long long token_stride, int q_at, int k_at, int v_at, int num_q,
                               int num_kv, int key_dim, int value_dim, int norm_mode, const void* q_weight,
                               const void* k_weight, int weight_dtype, float eps, const float* inv_freq,
                               int rot_dims, int pairing, const int* positions, const int* slots,
                               void* key_cache, void* value_cache, int page_size, const void* v_first,
                               long long v_first_stride, const void* blend, int tokens, int dtype,
                               const float* q_bias, const float* k_bias, const float* v_bias, void* stream) {
    if (tokens <= 0) return 0;
    if (v_bias && v_first) return TVB_BAD_ARGUMENT;          // a blended value has no bias of its own here
    if (key_dim <= 0 || key_dim > 64 * PREP_MAX_PAIRS || value_dim <= 0 || num_q <= 0 || num_kv < 0 ||
        num_q + 2 * num_kv > 65535 * PREP_WARPS || (slots && page_size <= 0) || norm_mode < 0 || norm_mode > 2 ||
        (norm_mode == PREP_NORM_WEIGHT && (!q_weight || !k_weight)) ||
        (inv_freq && (rot_dims <= 0 || rot_dims % 2 || rot_dims > key_dim || pairing < 0 || pairing > 1)) ||
        (v_first && !blend))
        return TVB_BAD_ARGUMENT;
    if ((int64_t)tokens * (num_q + 2 * num_kv) / 4 + 1 > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = dtype == TVB_BF16 && (key_dim == 16 || key_dim == 32 || key_dim == 64 || key_dim == 128 || key_dim == 256) &&
                      value_dim % 8 == 0 && q_at % 8 == 0 && k_at % 8 == 0 && v_at % 8 == 0 && token_stride % 8 == 0 &&
                      (uintptr_t)proj % 16 == 0 && (!inv_freq || pairing == PREP_PAIR_INTERLEAVED) &&
                      (!v_first || ((uintptr_t)v_first % 16 == 0 && v_first_stride % 8 == 0)) &&
                      (!slots || ((uintptr_t)key_cache % 16 == 0 && (uintptr_t)value_cache % 16 == 0));
    if (wide) {
#define WIDE(W)                                                                                                     \
    qkv_prepare_wide_kernel<W><<<(unsigned)tokens, PREP_WARPS * 32, 0, s>>>(                                        \
        (bf16*)proj, token_stride, q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim, norm_mode,                  \
        (const W*)q_weight, (const W*)k_weight, eps, inv_freq, rot_dims, positions, slots, (bf16*)key_cache,        \
        (bf16*)value_cache, page_size, (const bf16*)v_first, v_first_stride, (const bf16*)blend, q_bias, k_bias, v_bias)
        if (weight_dtype == TVB_F32) WIDE(float); else WIDE(bf16);
#undef WIDE
        return tvb_last_error();
    }
#define GO(T, W) return launch_prepare<T, W>(proj, token_stride, q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim, \
        norm_mode, q_weight, k_weight, eps, inv_freq, rot_dims, pairing, positions, slots, key_cache, value_cache,    \
        page_size, v_first, v_first_stride, blend, tokens, q_bias, k_bias, v_bias, s)
    if (dtype == TVB_F32 && weight_dtype == TVB_F32) GO(float, float);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16) GO(bf16, bf16);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32) GO(bf16, float);
#undef GO
    return TVB_BAD_ARGUMENT;
}

extern "C" int tvb_qkv_prepare(void* proj, long long token_stride, int q_at, int k_at, int v_at, int num_q,
                               int num_kv, int key_dim, int value_dim, int norm_mode, const void* q_weight,
                               const void* k_weight, int weight_dtype, float eps, const float* inv_freq,
                               int rot_dims, int pairing, const int* positions, const int* slots,
                               void* key_cache, void* value_cache, int page_size, const void* v_first,
                               long long v_first_stride, const void* blend, int tokens, int dtype, void* stream) {
    return tvb_qkv_prepare_biased(proj, token_stride, q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim, norm_mode,
                                  q_weight, k_weight, weight_dtype, eps, inv_freq, rot_dims, pairing, positions, slots,
                                  key_cache, value_cache, page_size, v_first, v_first_stride, blend, tokens, dtype,
                                  nullptr, nullptr, nullptr, stream);
}
