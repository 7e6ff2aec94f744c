// Pointwise steps around attention whose queries, keys and values come through low-rank latents,
// and around attention that normalises whole projections.  All arithmetic float32, one rounding
// to the storage type where a result is stored.
//
//   projection_norm   in place on segments of a packed projection row: v * rsqrt(mean(v^2) + eps) * w
//                     over the whole segment (all heads at once, weight of the segment's size), and,
//                     for segments that ask for it, times the query temperature
//                     1 + coef * ln(floor((p + 1) / every) + 1) of the token's position p; optionally the
//                     second segment (keys) and the values behind it go to the token's cache rows as well
//   latent_prepare    from a packed projection row [.. dq .. | .. dkv ..]: the query latent
//                     RMSnorm(dq) * w_q to a buffer; the key/value latent RMSnorm(dkv[:rank]) * w_kv and
//                     the rotated rest of dkv side by side, [latent | rotated], to the token's cache slot
//   rotate_heads      pairs (2i, 2i + 1) (or, with `halves`, (i, i + rot_dim / 2)) of a slice of every head turned by position * inv_freq[i],
//                     cosine and sine times `magnitude`, from one strided layout to another
//   head_product      out[t, h, j] = sum_k x[t, h, k] * w[h, j, k], optionally times sigmoid(gate[t, h, j]):
//                     one small product a head (the up-projections of latent attention, folded into the
//                     query and applied to the attended latents)
//   heads_place       the same result computed by a batched library product [h, t, j], put into [t, h, j]
//                     with the gate on the way (many tokens in bfloat16)
#include "common.cuh"

// ------------------------------------------------------------ projection_norm
struct NormSegment {
    int at, cols;
    const void* weight;
    int tempered;
};

// Where the second segment (the keys) and the values behind it go once they are ready: the token's rows
// of the paged caches [pages, num_kv, page, key_dim / value_dim].  `slots` null: nothing is stored.
struct CacheRows {
    const int* slots;
    void* key_cache;
    void* value_cache;
    int num_kv, key_dim, value_dim, page_size, v_at;
};

// A rotation behind the norm: in every head of `head_dim` elements of a segment the first `rot_dims` turn by
// position * inv_freq[pair], as pairs (2i, 2i + 1) or, with `halves`, (i, i + rot_dims / 2).  inv_freq null: none.
struct HeadRotation {
    const float* inv_freq;
    int rot_dims, halves, head_dim;
};

#define ROTATION_MAX_PAIRS 320      // pairs of a head that turn: their cosines and sines wait in shared memory

// element `d` of a head after the rotation, from the head's normalised values `head` (float32) and the token's
// cosines and sines a pair
__device__ __forceinline__ float rotated_element(const float* head, int d, const HeadRotation& rot,
                                                 const float* cos_s, const float* sin_s) {
    if (d >= rot.rot_dims) return head[d];
    const int half = rot.rot_dims >> 1;
    const bool first = rot.halves ? d < half : (d & 1) == 0;
    const int pair = rot.halves ? (first ? d : d - half) : d >> 1;
    const int other = rot.halves ? (first ? d + half : d - half) : (first ? d + 1 : d - 1);
    const float x = head[d], y = head[other], cosine = cos_s[pair], sine = sin_s[pair];
    return first ? __fsub_rn(__fmul_rn(x, cosine), __fmul_rn(y, sine)) : __fadd_rn(__fmul_rn(x, cosine), __fmul_rn(y, sine));
}

// eight consecutive weights (16-byte aligned) as float32
template <typename W> __device__ __forceinline__ void load_weights8(const W* p, float* w);
template <> __device__ __forceinline__ void load_weights8<bf16>(const bf16* p, float* w) {
    unpack_bf16x8(*reinterpret_cast<const uint4*>(p), w);
}
template <> __device__ __forceinline__ void load_weights8<float>(const float* p, float* w) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}

// The row waits in shared memory as float32 between the statistic and the result, so global memory is read
// once; WIDE: bfloat16 with every offset, size and stride a multiple of eight elements, eight values a thread
// and access.
template <typename T, typename W, bool WIDE>
__global__ void projection_norm_kernel(T* proj, int64_t stride, NormSegment first, NormSegment second,
                                       const int* __restrict__ positions, float eps, float coef, int every,
                                       CacheRows rows, HeadRotation rot) {
    extern __shared__ float row_values[];
    __shared__ float scratch[32];
    const NormSegment seg = blockIdx.y == 0 ? first : second;
    T* row = proj + (int64_t)blockIdx.x * stride + seg.at;
    const W* weight = (const W*)seg.weight;
    float part = 0.0f;
    if constexpr (WIDE) {
        for (int i = threadIdx.x * 8; i < seg.cols; i += blockDim.x * 8) {
            float v[8];
            unpack_bf16x8(ld_global_16(row + i), v);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                row_values[i + e] = v[e];
                part = __fmaf_rn(v[e], v[e], part);
            }
        }
    } else {
        for (int i = threadIdx.x; i < seg.cols; i += blockDim.x) {
            const float v = to_float<T>(row[i]);
            row_values[i] = v;
            part = __fmaf_rn(v, v, part);
        }
    }
    const float total = block_sum(part, scratch);
    const float inverse = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)seg.cols), eps)));
    float temperature = 1.0f;
    if (seg.tempered && every > 0) {
        const int p = max(positions[blockIdx.x], 0);
        temperature = __fmaf_rn(coef, logf((float)((p + 1) / every + 1)), 1.0f);
    }
    __shared__ float cos_s[ROTATION_MAX_PAIRS], sin_s[ROTATION_MAX_PAIRS];
    const bool turning = rot.inv_freq != nullptr;
    if (turning) {
        // the token's angles once, for all heads
        const float position = (float)max(positions[blockIdx.x], 0);
        for (int j = threadIdx.x; j < rot.rot_dims / 2; j += blockDim.x)
            sincosf(__fmul_rn(position, rot.inv_freq[j]), &sin_s[j], &cos_s[j]);
    }
    // neighbouring pairs lie inside a thread's eight values: they turn in registers (whole words turn or do not)
    const bool in_registers = WIDE && turning && !rot.halves && rot.rot_dims % 8 == 0;
    if (in_registers) __syncthreads();                               // the angles
    if (turning && !in_registers) {
        // the normalised row first, in shared memory, so that a pair's two elements are there whoever owns them
        if constexpr (WIDE) {
            for (int i = threadIdx.x * 8; i < seg.cols; i += blockDim.x * 8) {
                float w[8];
                load_weights8<W>(weight + i, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float o = __fmul_rn(__fmul_rn(row_values[i + e], inverse), w[e]);
                    if (seg.tempered) o = __fmul_rn(o, temperature);
                    row_values[i + e] = o;
                }
            }
        } else {
            for (int i = threadIdx.x; i < seg.cols; i += blockDim.x) {
                float o = __fmul_rn(__fmul_rn(row_values[i], inverse), to_float<W>(weight[i]));
                if (seg.tempered) o = __fmul_rn(o, temperature);
                row_values[i] = o;
            }
        }
        __syncthreads();
    }
    // the block of the second segment also stores: the normalised keys and the values to the token's cache rows
    const int slot = (blockIdx.y == 1 && rows.slots) ? rows.slots[blockIdx.x] : -1;
    const int64_t page_row = slot >= 0 ? (int64_t)(slot / rows.page_size) * rows.num_kv : 0;
    const int offset = slot >= 0 ? slot % rows.page_size : 0;
    if constexpr (WIDE) {
        for (int i = threadIdx.x * 8; i < seg.cols; i += blockDim.x * 8) {
            float w[8], o[8];
            if (in_registers) {
                load_weights8<W>(weight + i, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    o[e] = __fmul_rn(__fmul_rn(row_values[i + e], inverse), w[e]);
                    if (seg.tempered) o[e] = __fmul_rn(o[e], temperature);
                }
                const int d = i % rot.head_dim;
                if (d < rot.rot_dims) {
#pragma unroll
                    for (int pair = 0; pair < 4; ++pair) {
                        const float cosine = cos_s[(d >> 1) + pair], sine = sin_s[(d >> 1) + pair];
                        const float x = o[2 * pair], y = o[2 * pair + 1];
                        o[2 * pair] = __fsub_rn(__fmul_rn(x, cosine), __fmul_rn(y, sine));
                        o[2 * pair + 1] = __fadd_rn(__fmul_rn(y, cosine), __fmul_rn(x, sine));
                    }
                }
            } else if (turning) {
                const int d = i % rot.head_dim;                 // head_dim is a multiple of eight: one head a word
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = rotated_element(row_values + i - d, d + e, rot, cos_s, sin_s);
            } else {
                load_weights8<W>(weight + i, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    o[e] = __fmul_rn(__fmul_rn(row_values[i + e], inverse), w[e]);
                    if (seg.tempered) o[e] = __fmul_rn(o[e], temperature);
                }
            }
            const uint4 packed = pack_bf16x8(o);
            *reinterpret_cast<uint4*>(row + i) = packed;
            if (slot >= 0) {
                const int head = i / rows.key_dim, dim = i % rows.key_dim;      // key_dim is a multiple of eight
                *reinterpret_cast<uint4*>((bf16*)rows.key_cache +
                                          ((page_row + head) * rows.page_size + offset) * rows.key_dim + dim) = packed;
            }
        }
        if (slot >= 0) {
            const bf16* values = proj + (int64_t)blockIdx.x * stride + rows.v_at;
            for (int i = threadIdx.x * 8; i < rows.num_kv * rows.value_dim; i += blockDim.x * 8) {
                const int head = i / rows.value_dim, dim = i % rows.value_dim;
                *reinterpret_cast<uint4*>((bf16*)rows.value_cache +
                                          ((page_row + head) * rows.page_size + offset) * rows.value_dim + dim) =
                    ld_global_16(values + i);
            }
        }
    } else {
        for (int i = threadIdx.x; i < seg.cols; i += blockDim.x) {
            float o;
            if (turning) {
                const int d = i % rot.head_dim;
                o = rotated_element(row_values + i - d, d, rot, cos_s, sin_s);
            } else {
                o = __fmul_rn(__fmul_rn(row_values[i], inverse), to_float<W>(weight[i]));
                if (seg.tempered) o = __fmul_rn(o, temperature);
            }
            const T rounded = from_float<T>(o);
            row[i] = rounded;
            if (slot >= 0) {
                const int head = i / rows.key_dim, dim = i % rows.key_dim;
                ((T*)rows.key_cache)[((page_row + head) * rows.page_size + offset) * rows.key_dim + dim] = rounded;
            }
        }
        if (slot >= 0) {
            const T* values = proj + (int64_t)blockIdx.x * stride + rows.v_at;
            for (int i = threadIdx.x; i < rows.num_kv * rows.value_dim; i += blockDim.x) {
                const int head = i / rows.value_dim, dim = i % rows.value_dim;
                ((T*)rows.value_cache)[((page_row + head) * rows.page_size + offset) * rows.value_dim + dim] = values[i];
            }
        }
    }
}

// Two segments a launch (queries and keys); `second_cols` = 0 leaves the second out.  With `slots` the second
// segment is num_kv keys of key_dim elements: they go, normalised, to `key_cache`, and the num_kv values of
// value_dim elements from column `v_at` on go to `value_cache`, both at the token's slot (negative: nowhere).
//
// `inv_freq` (float32 [rot_dims / 2]): behind the norm the first `rot_dims` elements of every head of `head_dim`
// elements, in both segments, turn by the token's position (pairs (2i, 2i + 1), or with `halves` (i, i + rot_dims /
// 2)); the keys reach the cache turned.
extern "C" int tvb_projection_norm_rotate_store(void* proj, long long stride, int first_at, int first_cols,
                                                const void* first_weight, int first_tempered, int second_at,
                                                int second_cols, const void* second_weight, int second_tempered,
                                                int weight_dtype, const int* positions, float eps, float coef, int every,
                                                const int* slots, void* key_cache, void* value_cache, int num_kv,
                                                int key_dim, int value_dim, int page_size, int v_at, int tokens,
                                                int dtype, const float* inv_freq, int rot_dims, int halves,
                                                int head_dim, void* stream) {
    if (tokens <= 0) return 0;
    if (inv_freq && (!positions || rot_dims <= 0 || rot_dims % 2 || rot_dims / 2 > ROTATION_MAX_PAIRS || head_dim <= 0 || rot_dims > head_dim ||
                     first_cols % head_dim || second_cols % head_dim))
        return TVB_BAD_ARGUMENT;
    const HeadRotation rot{inv_freq, rot_dims, halves, head_dim};
    if (first_cols <= 0 || second_cols < 0 || !first_weight || (second_cols > 0 && !second_weight) ||
        ((first_tempered || second_tempered) && every > 0 && !positions))
        return TVB_BAD_ARGUMENT;
    if (slots && (!key_cache || !value_cache || num_kv <= 0 || key_dim <= 0 || value_dim <= 0 || page_size <= 0 ||
                  v_at < 0 || second_cols != num_kv * key_dim))
        return TVB_BAD_ARGUMENT;
    const CacheRows rows{slots, key_cache, value_cache, num_kv, key_dim, value_dim, page_size, v_at};
    cudaStream_t s = (cudaStream_t)stream;
    NormSegment first{first_at, first_cols, first_weight, first_tempered};
    NormSegment second{second_at, second_cols, second_weight, second_tempered};
    const int widest = first_cols > second_cols ? first_cols : second_cols;
    const size_t smem = (size_t)widest * sizeof(float);
    if (smem > 200 * 1024) return TVB_BAD_ARGUMENT;
    const bool wide = dtype == TVB_BF16 && (uintptr_t)proj % 16 == 0 && stride % 8 == 0 &&
                      first_at % 8 == 0 && first_cols % 8 == 0 && second_at % 8 == 0 && second_cols % 8 == 0 &&
                      (uintptr_t)first_weight % 16 == 0 && (!second_weight || (uintptr_t)second_weight % 16 == 0) &&
                      (!slots || (key_dim % 8 == 0 && value_dim % 8 == 0 && v_at % 8 == 0 &&
                                  (uintptr_t)key_cache % 16 == 0 && (uintptr_t)value_cache % 16 == 0)) &&
                      (!inv_freq || head_dim % 8 == 0);
    const int per_thread = wide ? 8 : 1;
    const int threads = widest / per_thread >= 512 ? 512 : (widest / per_thread >= 256 ? 256 : 128);
    for (int start = 0; start < tokens; start += 65535) {      // grid.x carries the tokens
        const int count = tokens - start < 65535 ? tokens - start : 65535;
        dim3 grid(count, second_cols > 0 ? 2 : 1);
        const int* p = positions ? positions + start : nullptr;
        CacheRows part = rows;
        if (part.slots) part.slots += start;
#define GO(T, W, WIDE)                                                                                         \
    do {                                                                                                       \
        auto kernel = projection_norm_kernel<T, W, WIDE>;                                                      \
        if (smem > 48 * 1024) {                                                                                \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                               \
        }                                                                                                      \
        kernel<<<grid, threads, smem, s>>>((T*)proj + (int64_t)start * stride, stride, first, second, p, eps,  \
                                           coef, every, part, rot);                                            \
    } while (0)
        if (dtype == TVB_F32 && weight_dtype == TVB_F32) GO(float, float, false);
        else if (dtype == TVB_BF16 && weight_dtype == TVB_BF16) { if (wide) GO(bf16, bf16, true); else GO(bf16, bf16, false); }
        else if (dtype == TVB_BF16 && weight_dtype == TVB_F32) { if (wide) GO(bf16, float, true); else GO(bf16, float, false); }
        else return TVB_BAD_ARGUMENT;
#undef GO
    }
    return tvb_last_error();
}

extern "C" int tvb_projection_norm_store(void* proj, long long stride, int first_at, int first_cols,
                                         const void* first_weight, int first_tempered, int second_at, int second_cols,
                                         const void* second_weight, int second_tempered, int weight_dtype,
                                         const int* positions, float eps, float coef, int every, const int* slots,
                                         void* key_cache, void* value_cache, int num_kv, int key_dim, int value_dim,
                                         int page_size, int v_at, int tokens, int dtype, void* stream) {
    return tvb_projection_norm_rotate_store(proj, stride, first_at, first_cols, first_weight, first_tempered, second_at,
                                            second_cols, second_weight, second_tempered, weight_dtype, positions, eps,
                                            coef, every, slots, key_cache, value_cache, num_kv, key_dim, value_dim,
                                            page_size, v_at, tokens, dtype, nullptr, 0, 0, 0, stream);
}

extern "C" int tvb_projection_norm(void* proj, long long stride, int first_at, int first_cols,
                                   const void* first_weight, int first_tempered, int second_at, int second_cols,
                                   const void* second_weight, int second_tempered, int weight_dtype,
                                   const int* positions, float eps, float coef, int every, int tokens, int dtype,
                                   void* stream) {
    return tvb_projection_norm_store(proj, stride, first_at, first_cols, first_weight, first_tempered, second_at,
                                     second_cols, second_weight, second_tempered, weight_dtype, positions, eps, coef,
                                     every, nullptr, nullptr, nullptr, 0, 0, 0, 0, 0, tokens, dtype, stream);
}

// ------------------------------------------------------------- latent_prepare
__device__ __forceinline__ void turn_pair(float u, float v, float angle, float magnitude, float& a, float& b) {
    float sine, cosine;
    sincosf(angle, &sine, &cosine);
    sine = __fmul_rn(sine, magnitude);
    cosine = __fmul_rn(cosine, magnitude);
    a = __fsub_rn(__fmul_rn(u, cosine), __fmul_rn(v, sine));
    b = __fadd_rn(__fmul_rn(v, cosine), __fmul_rn(u, sine));
}

template <typename T, typename W>
__global__ void latent_prepare_kernel(const T* proj, int64_t stride, int dq_at, int q_rank, const W* __restrict__ q_weight,
                                      T* __restrict__ q_latent, int64_t q_latent_stride, int dkv_at, int kv_rank,
                                      const W* __restrict__ kv_weight, int rot_dim, const float* __restrict__ inv_freq,
                                      float magnitude, const int* __restrict__ positions,
                                      const int* __restrict__ slots, T* __restrict__ cache, float eps, int halves) {
    __shared__ float scratch[32];
    const int token = blockIdx.x;
    const T* row = proj + (int64_t)token * stride;
    if (q_rank > 0) {
        float part = 0.0f;
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
            const float v = to_float<T>(row[dq_at + i]);
            part = __fmaf_rn(v, v, part);
        }
        const float total = block_sum(part, scratch);
        const float inverse = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)q_rank), eps)));
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
            q_latent[(int64_t)token * q_latent_stride + i] =
                from_float<T>(__fmul_rn(__fmul_rn(to_float<T>(row[dq_at + i]), inverse), to_float<W>(q_weight[i])));
    }
    const int slot = slots ? slots[token] : -1;
    if (slot < 0) return;                       // this run writes no cache, or a padding row
    T* dst = cache + (int64_t)slot * (kv_rank + rot_dim);
    float part = 0.0f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const float v = to_float<T>(row[dkv_at + i]);
        part = __fmaf_rn(v, v, part);
    }
    const float total = block_sum(part, scratch);
    const float inverse = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)kv_rank), eps)));
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
        dst[i] = from_float<T>(__fmul_rn(__fmul_rn(to_float<T>(row[dkv_at + i]), inverse), to_float<W>(kv_weight[i])));
    const float position = (float)positions[token];
    for (int i = threadIdx.x; i < rot_dim / 2; i += blockDim.x) {
        // pair i: elements (2i, 2i + 1), or with `halves` (i, i + rot_dim / 2)
        const int first = halves ? i : 2 * i, second = halves ? i + rot_dim / 2 : 2 * i + 1;
        float a, b;
        turn_pair(to_float<T>(row[dkv_at + kv_rank + first]), to_float<T>(row[dkv_at + kv_rank + second]),
                  __fmul_rn(position, inv_freq[i]), magnitude, a, b);
        dst[kv_rank + first] = from_float<T>(a);
        dst[kv_rank + second] = from_float<T>(b);
    }
}

// `cache`: rows of kv_rank + rot_dim per slot (one kv head); `slots` may be null (nothing is cached).
extern "C" int tvb_latent_prepare(const void* proj, long long stride, int dq_at, int q_rank, const void* q_weight,
                                  void* q_latent, long long q_latent_stride, int dkv_at, int kv_rank,
                                  const void* kv_weight, int weight_dtype, int rot_dim, const float* inv_freq,
                                  float magnitude, const int* positions, const int* slots, void* cache, float eps,
                                  int tokens, int dtype, int halves, void* stream) {
    if (tokens <= 0) return 0;
    if (q_rank < 0 || kv_rank <= 0 || rot_dim < 0 || rot_dim % 2 || !kv_weight || !positions ||
        (q_rank > 0 && (!q_weight || !q_latent)) || (rot_dim > 0 && !inv_freq) || (slots && !cache))
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int widest = q_rank > kv_rank ? q_rank : kv_rank;
    const int threads = widest >= 1024 ? 256 : (widest >= 256 ? 128 : 64);
#define GO(T, W) latent_prepare_kernel<T, W><<<tokens, threads, 0, s>>>(                                        \
        (const T*)proj, stride, dq_at, q_rank, (const W*)q_weight, (T*)q_latent, q_latent_stride, dkv_at,      \
        kv_rank, (const W*)kv_weight, rot_dim, inv_freq, magnitude, positions, slots, (T*)cache, eps, halves)
    if (dtype == TVB_F32 && weight_dtype == TVB_F32) GO(float, float);
    else if (dtype == TVB_BF16 && weight_dtype == TVB_BF16) GO(bf16, bf16);
    else if (dtype == TVB_BF16 && weight_dtype == TVB_F32) GO(bf16, float);
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}

// --------------------------------------------------------------- rotate_heads
template <typename T>
__global__ void rotate_heads_kernel(const T* src, int64_t src_token_stride, int64_t src_head_stride, T* dst,
                                    int64_t dst_token_stride, int64_t dst_head_stride, int heads, int rot_dim,
                                    const float* __restrict__ inv_freq, float magnitude,
                                    const int* __restrict__ positions, int64_t pairs, int halves) {
    const int64_t index = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= pairs) return;
    const int half = rot_dim / 2;
    const int i = (int)(index % half);
    const int head = (int)((index / half) % heads);
    const int64_t token = index / ((int64_t)half * heads);
    const int first = halves ? i : 2 * i, second = halves ? i + half : 2 * i + 1;
    const T* from = src + token * src_token_stride + head * src_head_stride;
    T* to = dst + token * dst_token_stride + head * dst_head_stride;
    float a, b;
    turn_pair(to_float<T>(from[first]), to_float<T>(from[second]),
              __fmul_rn((float)max(positions[token], 0), inv_freq[i]), magnitude, a, b);
    to[first] = from_float<T>(a);
    to[second] = from_float<T>(b);
}

extern "C" int tvb_rotate_heads(const void* src, long long src_token_stride, long long src_head_stride, void* dst,
                                long long dst_token_stride, long long dst_head_stride, int heads, int rot_dim,
                                const float* inv_freq, float magnitude, const int* positions, int tokens, int dtype,
                                int halves, void* stream) {
    if (tokens <= 0 || rot_dim == 0) return 0;
    if (heads <= 0 || rot_dim < 0 || rot_dim % 2 || !inv_freq || !positions) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t pairs = (int64_t)tokens * heads * (rot_dim / 2);
    const int64_t blocks = (pairs + 255) / 256;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
#define GO(T) rotate_heads_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(                                          \
        (const T*)src, src_token_stride, src_head_stride, (T*)dst, dst_token_stride, dst_head_stride, heads,    \
        rot_dim, inv_freq, magnitude, positions, pairs, halves)
    if (dtype == TVB_F32) GO(float);
    else if (dtype == TVB_BF16) GO(bf16);
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}

// --------------------------------------------------------------- head_product
// A block serves HP_TOKENS tokens of one head: their x rows wait in shared memory as float32, every
// warp takes output columns in turn, its lanes share the k of a weight row (coalesced) and the sums
// meet by shuffles.  The order of additions depends on k alone.
#define HP_TOKENS 8
#define HP_WARPS 8

#define HP_COLUMNS 32          // output columns a block takes (grid.z walks the rest)

template <typename T>
__global__ void head_product_kernel(const T* x, int64_t x_token_stride, int64_t x_head_stride,
                                    const T* __restrict__ w, T* out, int64_t out_token_stride,
                                    int64_t out_head_stride, const T* gate, int64_t gate_token_stride, int tokens,
                                    int n, int k) {
    extern __shared__ float x_rows[];                  // [HP_TOKENS][k]
    const int head = blockIdx.y;
    const int first = blockIdx.x * HP_TOKENS;
    const int count = min(HP_TOKENS, tokens - first);
    for (int i = threadIdx.x; i < HP_TOKENS * k; i += blockDim.x) {
        const int t = i / k, c = i % k;
        x_rows[i] = t < count ? to_float<T>(x[(int64_t)(first + t) * x_token_stride + head * x_head_stride + c]) : 0.0f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* w_head = w + (int64_t)head * n * k;
    const int last = min(n, (int)(blockIdx.z + 1) * HP_COLUMNS);
    for (int j = blockIdx.z * HP_COLUMNS + warp; j < last; j += HP_WARPS) {
        const T* w_row = w_head + (int64_t)j * k;
        float sums[HP_TOKENS];
#pragma unroll
        for (int t = 0; t < HP_TOKENS; ++t) sums[t] = 0.0f;
        for (int c = lane; c < k; c += 32) {
            const float wv = to_float<T>(w_row[c]);
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t) sums[t] = __fmaf_rn(x_rows[t * k + c], wv, sums[t]);
        }
#pragma unroll
        for (int t = 0; t < HP_TOKENS; ++t) sums[t] = warp_sum(sums[t]);
        if (lane < count) {
            float o = 0.0f;
#pragma unroll
            for (int t = 0; t < HP_TOKENS; ++t) if (t == lane) o = sums[t];
            if (gate) {
                const float g = to_float<T>(gate[(int64_t)(first + lane) * gate_token_stride + (int64_t)head * n + j]);
                o = __fmul_rn(o, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g))));
            }
            out[(int64_t)(first + lane) * out_token_stride + head * out_head_stride + j] = from_float<T>(o);
        }
    }
}

// x [tokens, heads, k] and out [tokens, heads, n] with strides of their own; w contiguous [heads, n, k];
// gate (optional) [tokens, heads * n] with a token stride.
extern "C" int tvb_head_product(const void* x, long long x_token_stride, long long x_head_stride, const void* w,
                                void* out, long long out_token_stride, long long out_head_stride, const void* gate,
                                long long gate_token_stride, int tokens, int heads, int n, int k, int dtype,
                                void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || n <= 0 || k <= 0) return TVB_BAD_ARGUMENT;
    const size_t smem = (size_t)HP_TOKENS * k * sizeof(float);
    if (smem > 48 * 1024) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid((tokens + HP_TOKENS - 1) / HP_TOKENS, heads, (n + HP_COLUMNS - 1) / HP_COLUMNS);
    if (grid.z > 65535) return TVB_BAD_ARGUMENT;
#define GO(T) head_product_kernel<T><<<grid, HP_WARPS * 32, smem, s>>>(                                          \
        (const T*)x, x_token_stride, x_head_stride, (const T*)w, (T*)out, out_token_stride, out_head_stride,     \
        (const T*)gate, gate_token_stride, tokens, n, k)
    if (dtype == TVB_F32) GO(float);
    else if (dtype == TVB_BF16) GO(bf16);
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}

// ---------------------------------------------------------------- heads_place
// dst[t, h, j] = src[h, t, j] (times sigmoid(gate[t, h * n + j])): the result of a batched library product,
// one batch a head, put where the next step reads it, with the gate on the way.
template <typename T>
__global__ void heads_place_kernel(const T* __restrict__ src, T* dst, int64_t dst_token_stride,
                                   int64_t dst_head_stride, const T* gate, int64_t gate_token_stride, int tokens,
                                   int heads, int n) {
    const int64_t index = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= (int64_t)tokens * heads * n) return;
    const int j = (int)(index % n);
    const int head = (int)((index / n) % heads);
    const int64_t token = index / ((int64_t)n * heads);
    float v = to_float<T>(src[((int64_t)head * tokens + token) * n + j]);
    if (gate) {
        const float g = to_float<T>(gate[token * gate_token_stride + (int64_t)head * n + j]);
        v = __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g))));
    }
    dst[token * dst_token_stride + head * dst_head_stride + j] = from_float<T>(v);
}

// bfloat16 with n, the strides and the addresses multiples of eight elements: eight values a thread and access
__global__ void heads_place_bf16x8_kernel(const bf16* __restrict__ src, bf16* dst, int64_t dst_token_stride,
                                          int64_t dst_head_stride, const bf16* gate, int64_t gate_token_stride,
                                          int tokens, int heads, int n) {
    const int64_t index = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int words = n / 8;
    if (index >= (int64_t)tokens * heads * words) return;
    const int j = (int)(index % words) * 8;
    const int head = (int)((index / words) % heads);
    const int64_t token = index / ((int64_t)words * heads);
    float v[8];
    unpack_bf16x8(ld_global_16(src + ((int64_t)head * tokens + token) * n + j), v);
    if (gate) {
        float g[8];
        unpack_bf16x8(ld_global_16(gate + token * gate_token_stride + (int64_t)head * n + j), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g[i]))));
    }
    *reinterpret_cast<uint4*>(dst + token * dst_token_stride + head * dst_head_stride + j) = pack_bf16x8(v);
}

extern "C" int tvb_heads_place(const void* src, void* dst, long long dst_token_stride, long long dst_head_stride,
                               const void* gate, long long gate_token_stride, int tokens, int heads, int n, int dtype,
                               void* stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || n <= 0) return TVB_BAD_ARGUMENT;
    const int64_t count = (int64_t)tokens * heads * n;
    const int64_t blocks = (count + 255) / 256;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == TVB_F32)
        heads_place_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((const float*)src, (float*)dst, dst_token_stride,
                                                                  dst_head_stride, (const float*)gate, gate_token_stride, tokens, heads, n);
    else if (dtype == TVB_BF16 && n % 8 == 0 && dst_token_stride % 8 == 0 && dst_head_stride % 8 == 0 &&
             (uintptr_t)src % 16 == 0 && (uintptr_t)dst % 16 == 0 &&
             (!gate || (gate_token_stride % 8 == 0 && (uintptr_t)gate % 16 == 0)))
        heads_place_bf16x8_kernel<<<(unsigned)((count / 8 + 255) / 256), 256, 0, s>>>(
            (const bf16*)src, (bf16*)dst, dst_token_stride, dst_head_stride, (const bf16*)gate, gate_token_stride,
            tokens, heads, n);
    else if (dtype == TVB_BF16)
        heads_place_kernel<bf16><<<(unsigned)blocks, 256, 0, s>>>((const bf16*)src, (bf16*)dst, dst_token_stride,
                                                                 dst_head_stride, (const bf16*)gate, gate_token_stride, tokens, heads, n);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}
