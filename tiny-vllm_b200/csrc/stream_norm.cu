// A residual stream kept in float32 whatever the storage type, and the kernels around it.
//
//   stream_norm   s' = s + (a + b)            (each of s, a, b optional; the sums in float32)
//                 y  = round_T(s' * rsqrt(mean(s'^2) + eps) * w)     (one rounding, at the end)
//                 One block per row.  With `gather` only the named rows are produced and the
//                 stream is not written (the last norm of a model, on the wanted rows).
//   gated_act     out = round_T(round_T(act(gate)) * up) for gate and up at two offsets of a
//                 strided row (a packed projection), act = SiLU or the tanh form of GELU
//   sum_pair      float32 a + b of two tensors of the storage type
//
// The statistics, the reciprocal root (a correctly rounded division of a correctly rounded
// root) and the product with the weight are float32; the order of additions inside a row
// depends on the width alone, so a row's result does not depend on the batch it is in.
#include "common.cuh"
#include <type_traits>

template <typename A, typename T, typename W>
__global__ void stream_norm_kernel(const float* stream_in, const A* add1, const A* add2,
                                   const W* __restrict__ weight, T* __restrict__ y, float* stream_out,
                                   const int* __restrict__ gather, int width, float eps) {
    extern __shared__ float row_values[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_launch_dependents();
    const int out_row = blockIdx.x;
    const int64_t in_row = gather ? gather[out_row] : out_row;
    const float* sr = stream_in ? stream_in + in_row * width : nullptr;
    const A* ar = add1 ? add1 + in_row * width : nullptr;
    const A* br = add2 ? add2 + in_row * width : nullptr;
    float part = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float update = ar ? to_float<A>(ar[i]) : 0.0f;
        if (br) update = __fadd_rn(update, to_float<A>(br[i]));
        const float v = sr ? ((ar || br) ? __fadd_rn(sr[i], update) : sr[i]) : update;
        row_values[i] = v;
        part = __fmaf_rn(v, v, part);
    }
    const float total = block_sum(part, scratch);
    const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)width), eps)));
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = row_values[i];
        if (stream_out && !gather) stream_out[(int64_t)out_row * width + i] = v;
        if (y) y[(int64_t)out_row * width + i] =
            from_float<T>(__fmul_rn(__fmul_rn(v, inverse_rms), to_float<W>(weight[i])));
    }
}

template <typename A, typename T, typename W>
static int launch_stream_norm(const float* stream_in, const void* add1, const void* add2, const void* weight,
                              void* y, float* stream_out, const int* gather, int rows, int width, float eps,
                              int pdl, cudaStream_t s) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TVB_BAD_ARGUMENT;
    auto kernel = stream_norm_kernel<A, T, W>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : (width >= 128 ? 128 : 32));
    TvbLaunch launch(dim3(rows), dim3(threads), smem, s, pdl);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, stream_in, (const A*)add1, (const A*)add2,
                                       (const W*)weight, (T*)y, stream_out, gather, width, eps);
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

// add_dtype: type of add1 / add2; dtype: type of y; weight_dtype: type of the norm weight.
extern "C" int tvb_stream_norm(const float* stream_in, const void* add1, const void* add2, int add_dtype,
                               const void* weight, int weight_dtype, void* y, int dtype, float* stream_out,
                               const int* gather, int rows, int width, float eps, int pdl, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || (!stream_in && !add1) || (add2 && !add1) || (y && !weight)) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
#define GO(A, T, W) return launch_stream_norm<A, T, W>(stream_in, add1, add2, weight, y, stream_out, gather, rows, width, eps, pdl, s)
    if (dtype == TVB_F32 && weight_dtype == TVB_F32 && add_dtype == TVB_F32) GO(float, float, float);
    if (dtype == TVB_F32 && weight_dtype == TVB_F32 && add_dtype == TVB_BF16) GO(bf16, float, float);   // a normed embedding
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16 && add_dtype == TVB_F32) GO(float, bf16, bf16);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16 && add_dtype == TVB_BF16) GO(bf16, bf16, bf16);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32 && add_dtype == TVB_F32) GO(float, bf16, float);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32 && add_dtype == TVB_BF16) GO(bf16, bf16, float);
#undef GO
    return TVB_BAD_ARGUMENT;
}

// ---------------------------------------------- a norm after a sublayer and the norm before the next
//   sandwich_norm   t  = y + scale[row] * x                    (the second term optional)
//                   s' = s + t * rsqrt(mean(t^2) + eps_post) * w_post     (without w_post: s' = s + t; without y: s' = s)
//                   out = round_T(s' * rsqrt(mean(s'^2) + eps_pre) * w_pre)   (without w_pre: no out)
//                   One block per row, all of it float32 with one rounding at the end.  A sublayer's output
//                   is normed before it joins the stream, and the stream is normed for the next sublayer, in
//                   one pass over the row.  With `gather` only the named rows are produced and the stream is
//                   not written.
//   add_scaled_rows y[row] += scale[row] * x[row]   (float32 y and scale, x of the storage type)
// four neighbouring values at once (16 bytes of float32, 8 of bfloat16), for rows whose width is a multiple of four
template <typename T> __device__ __forceinline__ void load4(const T* p, float* v);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float* v) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
    v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float* v);
template <> __device__ __forceinline__ void store4<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, const float* v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}

// VEC: values a thread moves at once, 4 (width a multiple of four, every pointer aligned to 4 values) or 1.  The
// order of a thread's additions differs between the two, a row's result by rounding only; which one runs depends
// on the width and the buffers' alignment, not on the batch.
template <typename Y, typename T, typename W, int VEC>
__global__ void sandwich_norm_kernel(const float* stream_in, const Y* y, const float* row_scale, const T* x,
                                     const W* __restrict__ post_weight, const W* __restrict__ pre_weight,
                                     T* __restrict__ out, float* stream_out, const int* __restrict__ gather,
                                     int width, float post_eps, float pre_eps) {
    extern __shared__ __align__(16) float row_values[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_launch_dependents();
    const int out_row = blockIdx.x;
    const int64_t in_row = gather ? gather[out_row] : out_row;
    const float* sr = stream_in + in_row * width;
    auto get = [](auto* p, float* v) {
        if constexpr (VEC == 4) load4(p, v);
        else v[0] = to_float<std::remove_cv_t<std::remove_pointer_t<decltype(p)>>>(*p);
    };
    float inverse_post = 1.0f;
    if (y) {
        const Y* yr = y + in_row * width;
        const T* xr = (x && row_scale) ? x + in_row * width : nullptr;
        const float scale = xr ? row_scale[in_row] : 0.0f;
        float part = 0.0f;
        for (int i = threadIdx.x * VEC; i < width; i += blockDim.x * VEC) {
            float t[VEC], a[VEC];
            get(yr + i, t);
            if (xr) get(xr + i, a);
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                if (xr) t[j] = __fmaf_rn(scale, a[j], t[j]);
                row_values[i + j] = t[j];
                part = __fmaf_rn(t[j], t[j], part);
            }
        }
        if (post_weight) {
            const float total = block_sum(part, scratch);
            inverse_post = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)width), post_eps)));
        }
    }
    float part = 0.0f;
    for (int i = threadIdx.x * VEC; i < width; i += blockDim.x * VEC) {          // a thread reads back only what it wrote
        float v[VEC], w[VEC];
        get(sr + i, v);
        if (y && post_weight) get(post_weight + i, w);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            if (y) {
                float t = row_values[i + j];
                if (post_weight) t = __fmul_rn(__fmul_rn(t, inverse_post), w[j]);
                v[j] = __fadd_rn(v[j], t);
            }
            row_values[i + j] = v[j];
            part = __fmaf_rn(v[j], v[j], part);
        }
    }
    float inverse_pre = 1.0f;
    if (pre_weight) {
        const float total = block_sum(part, scratch);
        inverse_pre = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)width), pre_eps)));
    }
    for (int i = threadIdx.x * VEC; i < width; i += blockDim.x * VEC) {
        float v[VEC], w[VEC], o[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = row_values[i + j];
        if (stream_out && !gather) {
            if constexpr (VEC == 4) store4(stream_out + (int64_t)out_row * width + i, v);
            else stream_out[(int64_t)out_row * width + i] = v[0];
        }
        if (pre_weight) {
            get(pre_weight + i, w);
#pragma unroll
            for (int j = 0; j < VEC; ++j) o[j] = __fmul_rn(__fmul_rn(v[j], inverse_pre), w[j]);
            if constexpr (VEC == 4) store4(out + (int64_t)out_row * width + i, o);
            else out[(int64_t)out_row * width + i] = from_float<T>(o[0]);
        }
    }
}

template <typename Y, typename T, typename W, int VEC>
static int launch_sandwich_norm_as(const float* stream_in, const void* y, const float* row_scale, const void* x,
                                   const void* post_weight, const void* pre_weight, void* out, float* stream_out,
                                   const int* gather, int rows, int width, float post_eps, float pre_eps, int pdl,
                                   cudaStream_t s) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TVB_BAD_ARGUMENT;
    auto kernel = sandwich_norm_kernel<Y, T, W, VEC>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int per = width / VEC;
    const int threads = per >= 2048 ? 512 : (per >= 512 ? 256 : (per >= 128 ? 128 : (per >= 64 ? 64 : 32)));
    TvbLaunch launch(dim3(rows), dim3(threads), smem, s, pdl);
    cudaError_t e = cudaLaunchKernelEx(&launch.config, kernel, stream_in, (const Y*)y, row_scale, (const T*)x,
                                       (const W*)post_weight, (const W*)pre_weight, (T*)out, stream_out, gather,
                                       width, post_eps, pre_eps);
    return e == cudaSuccess ? tvb_last_error() : (int)e;
}

template <typename Y, typename T, typename W>
static int launch_sandwich_norm(const float* stream_in, const void* y, const float* row_scale, const void* x,
                                const void* post_weight, const void* pre_weight, void* out, float* stream_out,
                                const int* gather, int rows, int width, float post_eps, float pre_eps, int pdl,
                                cudaStream_t s) {
    auto aligned = [](const void* p, size_t element) { return ((uintptr_t)p % (4 * element)) == 0; };
    const bool by_four = width % 4 == 0 && aligned(stream_in, 4) && aligned(y, sizeof(Y)) && aligned(x, sizeof(T)) &&
                         aligned(post_weight, sizeof(W)) && aligned(pre_weight, sizeof(W)) && aligned(out, sizeof(T)) &&
                         aligned(stream_out, 4);
    if (by_four)
        return launch_sandwich_norm_as<Y, T, W, 4>(stream_in, y, row_scale, x, post_weight, pre_weight, out, stream_out,
                                                   gather, rows, width, post_eps, pre_eps, pdl, s);
    return launch_sandwich_norm_as<Y, T, W, 1>(stream_in, y, row_scale, x, post_weight, pre_weight, out, stream_out,
                                               gather, rows, width, post_eps, pre_eps, pdl, s);
}

// y_dtype: type of y; dtype: type of x and out; weight_dtype: type of both norm weights.
extern "C" int tvb_sandwich_norm(const float* stream_in, const void* y, int y_dtype, const float* row_scale,
                                 const void* x, const void* post_weight, const void* pre_weight, int weight_dtype,
                                 void* out, int dtype, float* stream_out, const int* gather, int rows, int width,
                                 float post_eps, float pre_eps, int pdl, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || !stream_in || (pre_weight && !out) || (post_weight && !y) || ((row_scale != nullptr) != (x != nullptr)))
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
#define GO(Y, T, W) return launch_sandwich_norm<Y, T, W>(stream_in, y, row_scale, x, post_weight, pre_weight, out, \
                                                         stream_out, gather, rows, width, post_eps, pre_eps, pdl, s)
    if (dtype == TVB_F32 && weight_dtype == TVB_F32 && y_dtype == TVB_F32) GO(float, float, float);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16 && y_dtype == TVB_F32) GO(float, bf16, bf16);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32 && y_dtype == TVB_F32) GO(float, bf16, float);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16 && y_dtype == TVB_BF16) GO(bf16, bf16, bf16);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32 && y_dtype == TVB_BF16) GO(bf16, bf16, float);
#undef GO
    return TVB_BAD_ARGUMENT;
}

template <typename T>
__global__ void add_scaled_rows_kernel(float* __restrict__ y, const T* __restrict__ x, const float* __restrict__ scale,
                                       int width) {
    const int64_t row = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < width) y[row * width + i] = __fmaf_rn(scale[row], to_float<T>(x[row * width + i]), y[row * width + i]);
}

extern "C" int tvb_add_scaled_rows(float* y, const void* x, const float* scale, int rows, int width, int dtype,
                                   void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    for (int first = 0; first < rows; first += 65535) {
        const dim3 grid((width + 255) / 256, min(65535, rows - first));
        if (dtype == TVB_F32)
            add_scaled_rows_kernel<float><<<grid, 256, 0, s>>>(y + (int64_t)first * width, (const float*)x + (int64_t)first * width,
                                                              scale + first, width);
        else if (dtype == TVB_BF16)
            add_scaled_rows_kernel<bf16><<<grid, 256, 0, s>>>(y + (int64_t)first * width, (const bf16*)x + (int64_t)first * width,
                                                             scale + first, width);
        else return TVB_BAD_ARGUMENT;
    }
    return tvb_last_error();
}

// ------------------------------------------------------------ act(gate) * up
#define TVB_ACT_SILU 0
#define TVB_ACT_GELU_TANH 1

template <int ACT> __device__ __forceinline__ float activate(float z) {
    if (ACT == TVB_ACT_SILU) return __fdiv_rn(z, __fadd_rn(1.0f, expf(-z)));
    // 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
    const float inner = __fmul_rn(0.7978845608028654f, __fmaf_rn(__fmul_rn(0.044715f, z), __fmul_rn(z, z), z));
    return __fmul_rn(__fmul_rn(0.5f, z), __fadd_rn(1.0f, tanhf(inner)));
}

template <typename T, int ACT>
__global__ void gated_act_kernel(const T* in, int64_t in_stride, int gate_at, int up_at, T* __restrict__ out,
                                 int64_t out_stride, int inter) {
    const int64_t row = blockIdx.y;
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= inter) return;
    const T* src = in + row * in_stride;
    const float gate = to_float<T>(src[gate_at + col]);
    const float up = to_float<T>(src[up_at + col]);
    out[row * out_stride + col] = from_float<T>(__fmul_rn(round_to<T>(activate<ACT>(gate)), up));
}

// bfloat16 with every offset and stride a multiple of 8: eight values a thread, 16-byte accesses
template <int ACT>
__global__ void gated_act_bf16x8_kernel(const bf16* in, int64_t in_stride, int gate_at, int up_at,
                                        bf16* __restrict__ out, int64_t out_stride, int inter) {
    const int64_t row = blockIdx.y;
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (col >= inter) return;
    const bf16* src = in + row * in_stride;
    float gate[8], up[8], result[8];
    unpack_bf16x8(ld_global_16(src + gate_at + col), gate);
    unpack_bf16x8(ld_global_16(src + up_at + col), up);
#pragma unroll
    for (int i = 0; i < 8; ++i) result[i] = __fmul_rn(round_to<bf16>(activate<ACT>(gate[i])), up[i]);
    *reinterpret_cast<uint4*>(out + row * out_stride + col) = pack_bf16x8(result);
}

extern "C" int tvb_gated_act(const void* in, long long in_stride, int gate_at, int up_at, void* out,
                             long long out_stride, int rows, int inter, int act, int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (inter <= 0 || (act != TVB_ACT_SILU && act != TVB_ACT_GELU_TANH)) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const bool wide = dtype == TVB_BF16 && inter % 8 == 0 && gate_at % 8 == 0 && up_at % 8 == 0 &&
                      in_stride % 8 == 0 && out_stride % 8 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0;
    for (int first = 0; first < rows; first += 65535) {
        const int count = rows - first < 65535 ? rows - first : 65535;
        if (wide) {
            dim3 grid((inter / 8 + 127) / 128, count);
            const bf16* src = (const bf16*)in + (int64_t)first * in_stride;
            bf16* dst = (bf16*)out + (int64_t)first * out_stride;
            if (act == TVB_ACT_SILU)
                gated_act_bf16x8_kernel<TVB_ACT_SILU><<<grid, 128, 0, s>>>(src, in_stride, gate_at, up_at, dst, out_stride, inter);
            else
                gated_act_bf16x8_kernel<TVB_ACT_GELU_TANH><<<grid, 128, 0, s>>>(src, in_stride, gate_at, up_at, dst, out_stride, inter);
            continue;
        }
        dim3 grid((inter + 255) / 256, count);
#define GO(T, ACT)                                                                                   \
    gated_act_kernel<T, ACT><<<grid, 256, 0, s>>>((const T*)in + (int64_t)first * in_stride, in_stride, \
                                                  gate_at, up_at, (T*)out + (int64_t)first * out_stride, out_stride, inter)
        if (dtype == TVB_F32 && act == TVB_ACT_SILU) GO(float, TVB_ACT_SILU);
        else if (dtype == TVB_F32) GO(float, TVB_ACT_GELU_TANH);
        else if (dtype == TVB_BF16 && act == TVB_ACT_SILU) GO(bf16, TVB_ACT_SILU);
        else if (dtype == TVB_BF16) GO(bf16, TVB_ACT_GELU_TANH);
        else return TVB_BAD_ARGUMENT;
#undef GO
    }
    return tvb_last_error();
}

// ------------------------------------------------------------- float32 a + b
template <typename T>
__global__ void sum_pair_kernel(const T* a, const T* b, float* __restrict__ out, int64_t count) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = __fadd_rn(to_float<T>(a[i]), to_float<T>(b[i]));
}

extern "C" int tvb_sum_pair(const void* a, const void* b, float* out, long long count, int dtype, void* stream) {
    if (count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == TVB_F32) sum_pair_kernel<float><<<blocks, 256, 0, s>>>((const float*)a, (const float*)b, out, count);
    else if (dtype == TVB_BF16) sum_pair_kernel<bf16><<<blocks, 256, 0, s>>>((const bf16*)a, (const bf16*)b, out, count);
    else return TVB_BAD_ARGUMENT;
    return tvb_last_error();
}
