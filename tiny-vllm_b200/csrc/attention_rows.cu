// Paged causal attention, one warp per (query token, query head): the kernel of
// the float32 path and of every head size the tiled kernels do not take.
//
// The query at position p of a request attends the keys lo..p of that request
// (lo = max(0, p - window + 1) with a window, else 0) through the request's
// block table: key j of kv head g lies at row (table[j / page] * num_kv + g) * page + j % page
// of the cache [pages, num_kv, page, head_dim].  Query head
// h reads kv head h / (num_q / num_kv) (tinyvllm/kernels/paged_decode.cu:120).
// Scores, softmax and the output sum are float32 (:302-356, :457-465).
//
// Keys and values may differ in size (key_dim, value_dim; both up to 256).  With a window and
// keep_first > 0 the query also sees the keys 0..keep_first-1 that lie before its window.  An
// optional gate row g (same layout as the output) multiplies the output by sigmoid(g) before
// it is rounded and stored.
//
// Keys are processed in chunks of ATTN_CHUNK keys that start at absolute
// multiples of ATTN_CHUNK; every chunk gives a partial (max, sum, output) and the
// partials are merged in ascending order.  A row's arithmetic is therefore the
// same whether its chunks are walked by one warp (mode "rows", prompts) or by
// one warp per chunk with the partials in scratch memory and a merge kernel
// (mode "split", few rows with long contexts): the result at a position does not
// depend on how the tokens were cut into steps or batched.
#include "common.cuh"

#define ATTN_CHUNK 256
#define ATTN_MAX_DIMS 8      // head_dim <= 256: lane l owns dims l, l + 32, ...
#define ATTN_WIDE_DIMS 20    // the wide form: keys and values up to 640
#define ATTN_WARPS 4

template <int DIMS>
struct Partial {
    float max, sum;
    float out[DIMS];
};

// running (M, L, O) <- merge with a chunk's (m, l, o); explicit operations so that
// both callers compile to the same arithmetic.
template <int DIMS>
__device__ __forceinline__ void merge_partial(Partial<DIMS>& total, const Partial<DIMS>& part) {
    const float new_max = fmaxf(total.max, part.max);
    const float scale_total = total.max == -INFINITY ? 0.0f : expf(__fsub_rn(total.max, new_max));
    const float scale_part = part.max == -INFINITY ? 0.0f : expf(__fsub_rn(part.max, new_max));
    total.sum = __fadd_rn(__fmul_rn(total.sum, scale_total), __fmul_rn(part.sum, scale_part));
#pragma unroll
    for (int i = 0; i < DIMS; ++i)
        total.out[i] = __fadd_rn(__fmul_rn(total.out[i], scale_total), __fmul_rn(part.out[i], scale_part));
    total.max = new_max;
}


// q . k over one head in ascending order of the dimension; 16-byte loads when the
// head is a whole number of them (the order of additions is the same either way).
template <typename T>
__device__ __forceinline__ float dot_head(const float* __restrict__ q_shared, const T* __restrict__ k,
                                          int head_dim);
template <>
__device__ __forceinline__ float dot_head<float>(const float* __restrict__ q_shared,
                                                 const float* __restrict__ k, int head_dim) {
    float dot = 0.0f;
    if (head_dim % 4 == 0) {
        const float4* k4 = reinterpret_cast<const float4*>(k);
        for (int i = 0; i < head_dim / 4; ++i) {
            const float4 v = k4[i];
            dot = __fmaf_rn(q_shared[4 * i + 0], v.x, dot);
            dot = __fmaf_rn(q_shared[4 * i + 1], v.y, dot);
            dot = __fmaf_rn(q_shared[4 * i + 2], v.z, dot);
            dot = __fmaf_rn(q_shared[4 * i + 3], v.w, dot);
        }
    } else {
        for (int i = 0; i < head_dim; ++i) dot = __fmaf_rn(q_shared[i], k[i], dot);
    }
    return dot;
}
template <>
__device__ __forceinline__ float dot_head<bf16>(const float* __restrict__ q_shared,
                                                const bf16* __restrict__ k, int head_dim) {
    float dot = 0.0f;
    if (head_dim % 8 == 0) {
        const uint4* k8 = reinterpret_cast<const uint4*>(k);
        for (int i = 0; i < head_dim / 8; ++i) {
            const uint4 v = k8[i];
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                // a bfloat16 is the upper half of a float32
                dot = __fmaf_rn(q_shared[8 * i + 2 * w], __uint_as_float(words[w] << 16), dot);
                dot = __fmaf_rn(q_shared[8 * i + 2 * w + 1], __uint_as_float(words[w] & 0xffff0000u), dot);
            }
        }
    } else {
        for (int i = 0; i < head_dim; ++i) dot = __fmaf_rn(q_shared[i], __bfloat162float(k[i]), dot);
    }
    return dot;
}

// What is added to a score beside the scaled product: `slope` > 0 takes slope * (position - j) off the
// score of key j; `table` (or null) holds one learned number a distance, `stride` floats apart, and
// table[min(position - j, rows - 1) * stride] is added (all distances from rows - 1 on share the last).
struct ScoreBias {
    float slope;
    const float* table;
    int rows;
    int stride;
};

// The first key a query at `position` sees: the start of its window and of its own segment of
// `segment` positions (segments are counted from position 0), whichever is later.
__device__ __forceinline__ int first_visible(int position, int window, int segment) {
    int lo = window > 0 ? max(0, position - window + 1) : 0;
    if (segment > 0) lo = max(lo, position - position % segment);
    return lo;
}

// One chunk of keys [first, last] (inclusive, inside one ATTN_CHUNK block) for one row.
// `value_stride`: elements from one slot's value to the next (values may be a part of the key rows).
template <typename T, int DIMS>
__device__ __forceinline__ void attend_chunk(
    Partial<DIMS>& part, const float* __restrict__ q_shared, const T* __restrict__ key_cache,
    const T* __restrict__ value_cache, const int* __restrict__ table, int first, int last,
    int kv_head, int num_kv, int head_dim, int value_dim, int64_t value_stride, int page_size, float scale,
    const ScoreBias& bias, int position, int lane) {
    part.max = -INFINITY;
    part.sum = 0.0f;
#pragma unroll
    for (int i = 0; i < DIMS; ++i) part.out[i] = 0.0f;
    for (int base = first - first % 32; base <= last; base += 32) {
        const int j = base + lane;
        const bool valid = j >= first && j <= last;
        int64_t slot = 0;
        float score = -INFINITY;
        if (valid) {
            slot = ((int64_t)table[j / page_size] * num_kv + kv_head) * page_size + j % page_size;
            const T* k = key_cache + slot * head_dim;
            score = __fmul_rn(dot_head<T>(q_shared, k, head_dim), scale);
            if (bias.slope != 0.0f) score = __fsub_rn(score, __fmul_rn(bias.slope, (float)(position - j)));
            if (bias.table) score = __fadd_rn(score, bias.table[(int64_t)min(position - j, bias.rows - 1) * bias.stride]);
        }
        const float tile_max = warp_max(score);          // at least one key of a tile is valid
        const float new_max = fmaxf(part.max, tile_max);
        const float rescale = part.max == -INFINITY ? 0.0f : expf(__fsub_rn(part.max, new_max));
        const float p = valid ? expf(__fsub_rn(score, new_max)) : 0.0f;
        part.sum = __fadd_rn(__fmul_rn(part.sum, rescale), warp_sum(p));
#pragma unroll
        for (int i = 0; i < DIMS; ++i) part.out[i] = __fmul_rn(part.out[i], rescale);
        const int count = min(32, last - base + 1);
        for (int jj = max(0, first - base); jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int64_t sj = __shfl_sync(0xffffffffu, slot, jj);
            const T* v = value_cache + sj * value_stride;
#pragma unroll
            for (int i = 0; i < DIMS; ++i) {
                const int dim = lane + 32 * i;
                if (dim < value_dim) part.out[i] = __fmaf_rn(pj, to_float<T>(v[dim]), part.out[i]);
            }
        }
        part.max = new_max;
    }
}

// Everything of chunk `chunk` that the query at `position` sees: the kept first keys that fall
// into the chunk (they lie before lo), then the keys of the window.  Both pieces start from an
// empty partial and are merged in this order, whoever calls.
template <typename T, int DIMS>
__device__ __forceinline__ void attend_visible(
    Partial<DIMS>& part, const float* __restrict__ q_shared, const T* __restrict__ key_cache,
    const T* __restrict__ value_cache, const int* __restrict__ table, int chunk, int lo, int kept, int position,
    int kv_head, int num_kv, int head_dim, int value_dim, int64_t value_stride, int page_size, float scale,
    const ScoreBias& bias, int lane) {
    const int begin = chunk * ATTN_CHUNK, end = begin + ATTN_CHUNK - 1;
    const int first = max(lo, begin), last = min(position, end);
    if (kept > begin) {                                   // kept = min(keep_first, lo): keys 0..kept-1
        attend_chunk<T, DIMS>(part, q_shared, key_cache, value_cache, table, begin, min(kept - 1, end), kv_head,
                              num_kv, head_dim, value_dim, value_stride, page_size, scale, bias, position, lane);
        if (first <= last) {
            Partial<DIMS> more;
            attend_chunk<T, DIMS>(more, q_shared, key_cache, value_cache, table, first, last, kv_head, num_kv,
                                  head_dim, value_dim, value_stride, page_size, scale, bias, position, lane);
            merge_partial(part, more);
        }
        return;
    }
    attend_chunk<T, DIMS>(part, q_shared, key_cache, value_cache, table, first, last, kv_head, num_kv, head_dim,
                          value_dim, value_stride, page_size, scale, bias, position, lane);
}

// Whether the query sees anything of a chunk.
__device__ __forceinline__ bool chunk_visible(int chunk, int lo, int kept, int position) {
    const int begin = chunk * ATTN_CHUNK;
    return begin <= position && (begin + ATTN_CHUNK > lo || kept > begin);
}

__device__ __forceinline__ float gate_of(float g) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g))); }

// What the rows of one launch share beyond the sizes: `slopes` (one float a query head, or null):
// slope * (position - j) is taken off the score of key j; `sinks` (one float a query head, or null):
// exp(sink) is added to the softmax's denominator and to nothing else (nothing is attended for it); `gate_per_head`: the
// gate holds one number a head instead of one a value.
struct RowExtras {
    const float* slopes;
    const float* sinks;
    int gate_per_head;
    int64_t value_stride;
    const float* bias_table;      // float32 [bias_rows, num_q] (or null): a learned number a distance and head
    int bias_rows;
    int segment;                  // > 0: a query sees only the keys of its own segment of so many positions
};

// (M, L, O) of a finished row -> output: the sink joins the denominator, then division, gate, rounding.
template <typename T, int DIMS>
__device__ __forceinline__ void finish_row(Partial<DIMS>& total, const float* sinks, int head, const T* gate,
                                           int64_t gate_token_stride, int gate_per_head, int token, T* out_row,
                                           int value_dim, int lane) {
    float keep = 1.0f;
    if (sinks) {
        const float sink = sinks[head];
        const float top = fmaxf(total.max, sink);
        keep = expf(__fsub_rn(total.max, top));
        total.sum = __fadd_rn(__fmul_rn(total.sum, keep), expf(__fsub_rn(sink, top)));
    }
    const T* gate_row = nullptr;
    float head_gate = 1.0f;
    if (gate && gate_per_head) head_gate = gate_of(to_float<T>(gate[(int64_t)token * gate_token_stride + head]));
    else if (gate) gate_row = gate + (int64_t)token * gate_token_stride + (int64_t)head * value_dim;
#pragma unroll
    for (int i = 0; i < DIMS; ++i) {
        const int dim = lane + 32 * i;
        if (dim < value_dim) {
            float o = sinks ? __fdiv_rn(__fmul_rn(total.out[i], keep), total.sum) : __fdiv_rn(total.out[i], total.sum);
            if (gate_row) o = __fmul_rn(o, gate_of(to_float<T>(gate_row[dim])));
            else if (gate) o = __fmul_rn(o, head_gate);
            out_row[dim] = from_float<T>(o);
        }
    }
}

// mode rows: grid.x covers (token, head) rows, grid.y = 1, each warp walks all chunks.
// mode split: grid.y = chunk index; partials go to scratch.
template <typename T, bool SPLIT, int DIMS>
__global__ void paged_attention_rows_kernel(
    const T* __restrict__ q, int64_t q_token_stride, const T* __restrict__ key_cache,
    const T* __restrict__ value_cache, const int* __restrict__ block_tables, int table_stride,
    const int* __restrict__ token_row, const int* __restrict__ positions, T* __restrict__ out,
    int64_t out_token_stride, const T* gate, int64_t gate_token_stride,
    float* __restrict__ scratch, int max_chunks, int tokens, int num_q, int num_kv, int head_dim,
    int value_dim, int page_size, int window, int keep_first, float scale, RowExtras extras) {
    __shared__ float q_shared[ATTN_WARPS][DIMS * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * ATTN_WARPS + warp;
    if (row >= (int64_t)tokens * num_q) return;
    const int token = (int)(row / num_q), head = (int)(row % num_q);
    const int position = positions[token];
    const int request = token_row[token];
    T* out_row = out + (int64_t)token * out_token_stride + (int64_t)head * value_dim;
    if (request < 0 || position < 0) {            // padding row of a captured batch
        if (!SPLIT || blockIdx.y == 0)
            for (int i = lane; i < value_dim; i += 32) out_row[i] = from_float<T>(0.0f);
        return;
    }
    const int lo = first_visible(position, window, extras.segment);
    const int kept = min(keep_first, lo);
    const int last_chunk = position / ATTN_CHUNK;
    if (SPLIT && !chunk_visible(blockIdx.y, lo, kept, position)) return;
    const T* q_row = q + (int64_t)token * q_token_stride + (int64_t)head * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_shared[warp][i] = to_float<T>(q_row[i]);
    __syncwarp();
    const int* table = block_tables + (int64_t)request * table_stride;
    const int kv_head = head / (num_q / num_kv);
    const ScoreBias bias{extras.slopes ? extras.slopes[head] : 0.0f,
                         extras.bias_table ? extras.bias_table + head : nullptr, extras.bias_rows, num_q};

    if (SPLIT) {
        const int chunk = blockIdx.y;
        Partial<DIMS> part;
        attend_visible<T, DIMS>(part, q_shared[warp], key_cache, value_cache, table, chunk, lo, kept, position,
                                kv_head, num_kv, head_dim, value_dim, extras.value_stride, page_size, scale, bias,
                                lane);
        float* dst = scratch + (row * max_chunks + chunk) * (int64_t)(value_dim + 2);
        if (lane == 0) { dst[0] = part.max; dst[1] = part.sum; }
#pragma unroll
        for (int i = 0; i < DIMS; ++i) {
            const int dim = lane + 32 * i;
            if (dim < value_dim) dst[2 + dim] = part.out[i];
        }
    } else {
        Partial<DIMS> total;
        total.max = -INFINITY;
        total.sum = 0.0f;
#pragma unroll
        for (int i = 0; i < DIMS; ++i) total.out[i] = 0.0f;
        for (int chunk = 0; chunk <= last_chunk; ++chunk) {
            if (!chunk_visible(chunk, lo, kept, position)) continue;
            Partial<DIMS> part;
            attend_visible<T, DIMS>(part, q_shared[warp], key_cache, value_cache, table, chunk, lo, kept, position,
                                    kv_head, num_kv, head_dim, value_dim, extras.value_stride, page_size, scale,
                                    bias, lane);
            merge_partial(total, part);
        }
        finish_row<T, DIMS>(total, extras.sinks, head, gate, gate_token_stride, extras.gate_per_head, token,
                            out_row, value_dim, lane);
    }
}

template <typename T, int DIMS>
__global__ void merge_attention_rows_kernel(const float* __restrict__ scratch, int max_chunks,
                                            const int* __restrict__ token_row,
                                            const int* __restrict__ positions, T* __restrict__ out,
                                            int64_t out_token_stride, const T* gate, int64_t gate_token_stride,
                                            int tokens, int num_q, int head_dim, int window, int keep_first,
                                            RowExtras extras) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * ATTN_WARPS + warp;
    if (row >= (int64_t)tokens * num_q) return;
    const int token = (int)(row / num_q), head = (int)(row % num_q);
    const int position = positions[token];
    if (token_row[token] < 0 || position < 0) return;     // zeros were written by the first kernel
    const int lo = first_visible(position, window, extras.segment);
    const int kept = min(keep_first, lo);
    T* out_row = out + (int64_t)token * out_token_stride + (int64_t)head * head_dim;
    Partial<DIMS> total;
    total.max = -INFINITY;
    total.sum = 0.0f;
#pragma unroll
    for (int i = 0; i < DIMS; ++i) total.out[i] = 0.0f;
    // The scratch holds max_chunks partials a row.  A caller whose max_chunks is too small for this
    // row's position gets the row as NaN: the first kernel wrote no partial beyond max_chunks - 1,
    // and reading on would take the next row's (or leave the buffer).
    const int last_chunk = position / ATTN_CHUNK;
    if (last_chunk >= max_chunks) {
        T* bad_row = out_row;
        for (int dim = lane; dim < head_dim; dim += 32) bad_row[dim] = from_float<T>(__int_as_float(0x7fc00000));
        return;
    }
    for (int chunk = 0; chunk <= last_chunk; ++chunk) {
        if (!chunk_visible(chunk, lo, kept, position)) continue;
        const float* src = scratch + (row * max_chunks + chunk) * (int64_t)(head_dim + 2);
        Partial<DIMS> part;
        part.max = src[0];
        part.sum = src[1];
#pragma unroll
        for (int i = 0; i < DIMS; ++i) {
            const int dim = lane + 32 * i;
            part.out[i] = dim < head_dim ? src[2 + dim] : 0.0f;
        }
        merge_partial(total, part);
    }
    finish_row<T, DIMS>(total, extras.sinks, head, gate, gate_token_stride, extras.gate_per_head, token, out_row,
                        head_dim, lane);
}

extern "C" int tvb_attention_chunk_keys() { return ATTN_CHUNK; }

// scratch floats the split mode needs: tokens * num_q * max_chunks * (head_dim + 2)
extern "C" long long tvb_attention_rows_scratch_floats(int tokens, int num_q, int head_dim, int max_chunks) {
    return (long long)tokens * num_q * max_chunks * (head_dim + 2);
}

template <typename T, int DIMS>
static void launch_rows(const void* q, long long q_token_stride, const void* key_cache, const void* value_cache,
                        const int* block_tables, int table_stride, const int* token_row, const int* positions,
                        void* out, long long out_token_stride, const void* gate, long long gate_token_stride,
                        float* scratch, int max_chunks, int tokens, int num_q, int num_kv, int head_dim,
                        int value_dim, int page_size, int window, int keep_first, float scale, RowExtras extras,
                        unsigned blocks, cudaStream_t s) {
    dim3 grid(blocks, max_chunks > 0 ? max_chunks : 1);
    if (max_chunks > 0) {
        paged_attention_rows_kernel<T, true, DIMS><<<grid, ATTN_WARPS * 32, 0, s>>>(
            (const T*)q, q_token_stride, (const T*)key_cache, (const T*)value_cache, block_tables, table_stride,
            token_row, positions, (T*)out, out_token_stride, (const T*)gate, gate_token_stride, scratch, max_chunks,
            tokens, num_q, num_kv, head_dim, value_dim, page_size, window, keep_first, scale, extras);
        merge_attention_rows_kernel<T, DIMS><<<blocks, ATTN_WARPS * 32, 0, s>>>(
            scratch, max_chunks, token_row, positions, (T*)out, out_token_stride, (const T*)gate, gate_token_stride,
            tokens, num_q, value_dim, window, keep_first, extras);
    } else {
        paged_attention_rows_kernel<T, false, DIMS><<<grid, ATTN_WARPS * 32, 0, s>>>(
            (const T*)q, q_token_stride, (const T*)key_cache, (const T*)value_cache, block_tables, table_stride,
            token_row, positions, (T*)out, out_token_stride, (const T*)gate, gate_token_stride, scratch, max_chunks,
            tokens, num_q, num_kv, head_dim, value_dim, page_size, window, keep_first, scale, extras);
    }
}

// max_chunks = 0 selects mode rows (no scratch).  Otherwise max_chunks must be at
// least ceil((largest position + 1) / ATTN_CHUNK) of the batch and scratch must hold
// tokens * num_q * max_chunks * (value_dim + 2) floats.  The host cannot see the positions:
// a row whose position needs more chunks than max_chunks is written as NaN (and nothing
// outside the stated scratch is read or written).
// The widest form: keys `head_dim` and values `value_dim` wide (up to 640), the first `keep_first`
// keys seen from behind a window, output rows `out_token_stride` apart, an optional gate with a stride
// of its own, one number a value or (`gate_per_head`) one a head, a distance bias (`slopes`), a sink in
// the denominator (`sinks`), and values that lie `value_stride` elements apart (0: value_dim), which
// lets them be a part of the key rows.
// `bias_table` (float32 [bias_rows, num_q], or null): table[min(p - j, bias_rows - 1), h] is added to the
// score of key j; `segment` > 0: the query at p sees only keys from p - p % segment on.
extern "C" int tvb_attention_rows_masked(const void* q, long long q_token_stride, const void* key_cache,
                                         const void* value_cache, long long value_stride, const int* block_tables,
                                         int table_stride, const int* token_row, const int* positions, void* out,
                                         long long out_token_stride, const void* gate, long long gate_token_stride,
                                         int gate_per_head, const float* slopes, const float* sinks,
                                         const float* bias_table, int bias_rows, int segment,
                                         float* scratch, int max_chunks, int tokens, int num_q, int num_kv,
                                         int head_dim, int value_dim, int page_size, int window, int keep_first,
                                         float scale, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (segment < 0 || (bias_table && bias_rows <= 0)) return TVB_BAD_ARGUMENT;
    if (head_dim <= 0 || head_dim > 32 * ATTN_WIDE_DIMS || value_dim <= 0 || value_dim > 32 * ATTN_WIDE_DIMS ||
        num_q <= 0 || num_kv <= 0 || keep_first < 0 || value_stride < 0 ||
        num_q % num_kv || page_size <= 0 || max_chunks < 0 || max_chunks > 65535 ||
        (max_chunks > 0 && !scratch))
        return TVB_BAD_ARGUMENT;
    const int64_t rows = (int64_t)tokens * num_q;
    const int64_t blocks = (rows + ATTN_WARPS - 1) / ATTN_WARPS;
    if (blocks > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    RowExtras extras{slopes, sinks, gate_per_head, value_stride > 0 ? value_stride : value_dim,
                     bias_table, bias_rows, segment};
    const bool wide = head_dim > 32 * ATTN_MAX_DIMS || value_dim > 32 * ATTN_MAX_DIMS;
#define LAUNCH_ROWS(T, DIMS)                                                                             \
    launch_rows<T, DIMS>(q, q_token_stride, key_cache, value_cache, block_tables, table_stride, token_row, \
                         positions, out, out_token_stride, gate, gate_token_stride, scratch, max_chunks,   \
                         tokens, num_q, num_kv, head_dim, value_dim, page_size, window, keep_first, scale, \
                         extras, (unsigned)blocks, s)
    if (dtype == TVB_F32) { if (wide) LAUNCH_ROWS(float, ATTN_WIDE_DIMS); else LAUNCH_ROWS(float, ATTN_MAX_DIMS); }
    else if (dtype == TVB_BF16) { if (wide) LAUNCH_ROWS(bf16, ATTN_WIDE_DIMS); else LAUNCH_ROWS(bf16, ATTN_MAX_DIMS); }
    else return TVB_BAD_ARGUMENT;
#undef LAUNCH_ROWS
    return tvb_last_error();
}

extern "C" int tvb_attention_rows_biased(const void* q, long long q_token_stride, const void* key_cache,
                                         const void* value_cache, long long value_stride, const int* block_tables,
                                         int table_stride, const int* token_row, const int* positions, void* out,
                                         long long out_token_stride, const void* gate, long long gate_token_stride,
                                         int gate_per_head, const float* slopes, const float* sinks,
                                         float* scratch, int max_chunks, int tokens, int num_q, int num_kv,
                                         int head_dim, int value_dim, int page_size, int window, int keep_first,
                                         float scale, int dtype, void* stream) {
    return tvb_attention_rows_masked(q, q_token_stride, key_cache, value_cache, value_stride, block_tables,
                                     table_stride, token_row, positions, out, out_token_stride, gate,
                                     gate_token_stride, gate_per_head, slopes, sinks, nullptr, 0, 0, scratch,
                                     max_chunks, tokens, num_q, num_kv, head_dim, value_dim, page_size, window,
                                     keep_first, scale, dtype, stream);
}

extern "C" int tvb_attention_rows_general(const void* q, long long q_token_stride, const void* key_cache,
                                          const void* value_cache, const int* block_tables, int table_stride,
                                          const int* token_row, const int* positions, void* out,
                                          long long out_token_stride, const void* gate, long long gate_token_stride,
                                          float* scratch, int max_chunks, int tokens, int num_q, int num_kv,
                                          int head_dim, int value_dim, int page_size, int window, int keep_first,
                                          float scale, int dtype, void* stream) {
    if (head_dim > 32 * ATTN_MAX_DIMS || value_dim > 32 * ATTN_MAX_DIMS) return TVB_BAD_ARGUMENT;
    return tvb_attention_rows_biased(q, q_token_stride, key_cache, value_cache, 0, block_tables, table_stride,
                                     token_row, positions, out, out_token_stride, gate, gate_token_stride, 0,
                                     nullptr, nullptr, scratch, max_chunks, tokens, num_q, num_kv, head_dim,
                                     value_dim, page_size, window, keep_first, scale, dtype, stream);
}

extern "C" int tvb_attention_rows(const void* q, long long q_token_stride, const void* key_cache,
                                  const void* value_cache, const int* block_tables, int table_stride,
                                  const int* token_row, const int* positions, void* out,
                                  float* scratch, int max_chunks, int tokens, int num_q, int num_kv,
                                  int head_dim, int page_size, int window, float scale, int dtype,
                                  void* stream) {
    return tvb_attention_rows_general(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                                      token_row, positions, out, (long long)num_q * head_dim, nullptr, 0, scratch,
                                      max_chunks, tokens, num_q, num_kv, head_dim, head_dim, page_size, window, 0,
                                      scale, dtype, stream);
}

// ------------------------------------------------ entry point that allocates nothing
// See attention_rows_static.h for who needs this and how to use it.
#include "attention_rows_static.h"

// The scratch of the split mode, held by every GPU that loads this library until exit.
static __device__ __align__(256) float tvb_static_scratch[TVB_STATIC_SCRATCH_FLOATS];

// In host code `tvb_static_scratch` is only a stand-in for the symbol, not a device address:
// the address is asked for once per device, with that device current, and kept here.
#define TVB_STATIC_MAX_DEVICES 64
static float* tvb_static_scratch_address[TVB_STATIC_MAX_DEVICES];

static int tvb_static_scratch_of_current_device(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= TVB_STATIC_MAX_DEVICES) return TVB_BAD_ARGUMENT;
    if (!tvb_static_scratch_address[device]) {
        float* found = nullptr;
        e = cudaGetSymbolAddress((void**)&found, tvb_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!found) return (int)cudaErrorInvalidSymbol;
        tvb_static_scratch_address[device] = found;
    }
    *address = tvb_static_scratch_address[device];
    return 0;
}

extern "C" long long tvb_attention_rows_static_capacity(void) { return TVB_STATIC_SCRATCH_FLOATS; }

extern "C" const char* tvb_attention_rows_static_error(int code) {
    if (code == 0) return "ok";
    if (code == TVB_STATIC_SCRATCH_TOO_SMALL)
        return "the partials of this batch (tokens * num_q * max_chunks * (head_dim + 2) floats) do not fit "
               "into the library's built-in scratch of 4 Mi floats; use tvb_attention_rows with a buffer of "
               "your own, or fewer tokens per call";
    if (code == TVB_BAD_ARGUMENT)
        return "sizes this kernel does not take (or max_chunks == 0, which needs no scratch: call "
               "tvb_attention_rows)";
    return cudaGetErrorString((cudaError_t)code);
}

extern "C" int tvb_attention_rows_static(const void* q, long long q_token_stride, const void* key_cache,
                                         const void* value_cache, const int* block_tables, int table_stride,
                                         const int* token_row, const int* positions, void* out,
                                         int max_chunks, int tokens, int num_q, int num_kv, int head_dim,
                                         int page_size, int window, float scale, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    // bounds first, so that the product below cannot overflow
    if (max_chunks <= 0 || max_chunks > 65535 || num_q <= 0 || num_q > 65535 || head_dim <= 0 ||
        head_dim > 32 * ATTN_MAX_DIMS)
        return TVB_BAD_ARGUMENT;
    if (tokens > TVB_STATIC_SCRATCH_FLOATS) return TVB_STATIC_SCRATCH_TOO_SMALL;      // every token needs floats
    if (tvb_attention_rows_scratch_floats(tokens, num_q, head_dim, max_chunks) > TVB_STATIC_SCRATCH_FLOATS)
        return TVB_STATIC_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    const int status = tvb_static_scratch_of_current_device(&scratch);
    if (status != 0) return status;
    // the launcher below only checks sizes and launches the two kernels
    return tvb_attention_rows(q, q_token_stride, key_cache, value_cache, block_tables, table_stride,
                              token_row, positions, out, scratch, max_chunks, tokens, num_q, num_kv,
                              head_dim, page_size, window, scale, dtype, stream);
}
