// Routing of a mixture of experts and the experts' activation in one pass.
//
// Per token: the `top` experts with the largest router logits (float32; of equal logits the lower
// index wins) get the softmax over their logits alone as weights, all others weight 0.  Then the
// packed up-projection [experts * ff | shared_ff] of the token becomes the input of the packed
// down-projection: column c of expert e holds act(up[c]) * weight_e (exactly 0 for an expert that
// was not chosen), the shared expert's columns hold act(up[c]); act is relu(z)^2 or SiLU.  The
// down-projection over all columns at once is then the weighted sum of the chosen experts' outputs
// plus the shared expert's.  Weights and activation are float32, one rounding to the storage type.
//
// A second form (route_gated_act) serves routers that score with a sigmoid: see its kernel.
#include "common.cuh"

#define ROUTE_MAX_EXPERTS 1024
#define TVB_ACT_RELU2 0
#define TVB_ACT_SILU_PLAIN 1

template <int ACT> __device__ __forceinline__ float expert_act(float z) {
    if (ACT == TVB_ACT_RELU2) {
        const float r = fmaxf(z, 0.0f);
        return __fmul_rn(r, r);
    }
    return __fdiv_rn(z, __fadd_rn(1.0f, expf(-z)));
}

template <typename T, int ACT, bool WIDE>
__global__ void route_act_kernel(const float* __restrict__ logits, int64_t logits_stride, const T* up,
                                 int64_t up_stride, T* __restrict__ out, int64_t out_stride,
                                 float* __restrict__ weights_out, int experts, int top, int ff, int shared_ff) {
    __shared__ float share[ROUTE_MAX_EXPERTS];       // the weight of every expert, 0 if not chosen
    __shared__ float value[ROUTE_MAX_EXPERTS];
    const int64_t token = blockIdx.x;
    const float* z = logits + token * logits_stride;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        value[e] = z[e];
        share[e] = 0.0f;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float best_of_all = 0.0f, sum = 0.0f;
        for (int round = 0; round < top; ++round) {
            float best = -INFINITY;
            int where = ROUTE_MAX_EXPERTS;
            for (int e = lane; e < experts; e += 32)
                if (value[e] > best) { best = value[e]; where = e; }
#pragma unroll
            for (int delta = 16; delta > 0; delta >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, best, delta);
                const int other_where = __shfl_xor_sync(0xffffffffu, where, delta);
                if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
            }
            if (where >= experts) break;                // fewer experts than `top`
            if (round == 0) best_of_all = best;
            const float e_weight = expf(__fsub_rn(best, best_of_all));
            sum = __fadd_rn(sum, e_weight);
            if (lane == 0) { share[where] = e_weight; value[where] = -INFINITY; }
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32) share[e] = __fdiv_rn(share[e], sum);
    }
    __syncthreads();
    if (weights_out && blockIdx.y == 0)
        for (int e = threadIdx.x; e < experts; e += blockDim.x) weights_out[token * experts + e] = share[e];
    const T* src = up + token * up_stride;
    T* dst = out + token * out_stride;
    const int routed = experts * ff;
    // grid.y shares the columns: every block finds the token's experts for itself (a few dozen logits)
    int per_block = (routed + shared_ff + gridDim.y - 1) / gridDim.y;
    if (WIDE) per_block = (per_block + 7) / 8 * 8;
    const int begin = blockIdx.y * per_block, end = min(routed + shared_ff, begin + per_block);
    if constexpr (WIDE) {
        // bfloat16 rows whose pieces are whole 16-byte words: eight columns a thread and access (an expert's
        // columns are a multiple of eight, so a word never straddles two experts)
        for (int c = begin + threadIdx.x * 8; c < end; c += blockDim.x * 8) {
            float v[8], o[8];
            unpack_bf16x8(ld_global_16(src + c), v);
            const float weight = c < routed ? share[c / ff] : 1.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a = expert_act<ACT>(v[i]);
                o[i] = c < routed ? __fmul_rn(a, weight) : a;
            }
            *reinterpret_cast<uint4*>(dst + c) = pack_bf16x8(o);
        }
    } else {
        for (int c = begin + threadIdx.x; c < end; c += blockDim.x) {
            const float a = expert_act<ACT>(to_float<T>(src[c]));
            dst[c] = from_float<T>(c < routed ? __fmul_rn(a, share[c / ff]) : a);
        }
    }
}

// logits [tokens, experts] float32; up and out [tokens, experts * ff + shared_ff] with row strides;
// weights_out (optional) [tokens, experts] float32 receives every expert's weight.
extern "C" int tvb_route_act(const float* logits, long long logits_stride, const void* up, long long up_stride,
                             void* out, long long out_stride, float* weights_out, int tokens, int experts, int top,
                             int ff, int shared_ff, int act, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top <= 0 || ff <= 0 || shared_ff < 0 ||
        (act != TVB_ACT_RELU2 && act != TVB_ACT_SILU_PLAIN))
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const long long columns = (long long)experts * ff + shared_ff;
    const int threads = 256;
    // few tokens: the columns of a token are spread over several blocks, so that the GPU has some 300 of them
    long long split = tokens >= 296 ? 1 : (296 + tokens - 1) / tokens;
    const long long most = (columns + 4 * threads - 1) / (4 * threads);
    if (split > most) split = most;
    if (split > 65535) split = 65535;
    const dim3 grid(tokens, (unsigned)split);
    const bool wide = dtype == TVB_BF16 && ff % 8 == 0 && shared_ff % 8 == 0 && up_stride % 8 == 0 &&
                      out_stride % 8 == 0 && (uintptr_t)up % 16 == 0 && (uintptr_t)out % 16 == 0;
#define GO(T, ACT, WIDE) route_act_kernel<T, ACT, WIDE><<<grid, threads, 0, s>>>(                          \
        logits, logits_stride, (const T*)up, up_stride, (T*)out, out_stride, weights_out, experts, top, ff, shared_ff)
    if (dtype == TVB_F32 && act == TVB_ACT_RELU2) GO(float, TVB_ACT_RELU2, false);
    else if (dtype == TVB_F32) GO(float, TVB_ACT_SILU_PLAIN, false);
    else if (dtype == TVB_BF16 && act == TVB_ACT_RELU2) { if (wide) GO(bf16, TVB_ACT_RELU2, true); else GO(bf16, TVB_ACT_RELU2, false); }
    else if (dtype == TVB_BF16) { if (wide) GO(bf16, TVB_ACT_SILU_PLAIN, true); else GO(bf16, TVB_ACT_SILU_PLAIN, false); }
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}


// ------------------------------------------------------------------------------------------------
// Sigmoid routing with a choice correction and groups of experts, and gated experts with limits.
//
// Per token, from router logits z (float32): s_e = sigmoid(z_e); the choice score is s_e + correction_e
// (`correction` may be null).  With `groups` > 1 the experts form that many equal groups of neighbours;
// a group's score is the sum of its two largest choice scores (of its one, if it has one expert), and
// only experts of the `keep` best groups can be chosen.  The `top` experts with the largest choice
// scores are chosen (of equal scores the lower index wins); their weights are s_e / (sum of the chosen
// s + 1e-20) * route_scale.
//
// The packed projection of a token holds [gate_e | up_e] (ff columns each) expert after expert, then
// [gate | up] of the shared expert (shared_ff each).  With g = min(gate, limit) and u = clamp(up,
// -limit, limit) an expert's inner activation is g * sigmoid(alpha * g) * (u + 1); column c of expert
// e of the output holds it times the expert's weight (exactly 0 if the expert was not chosen).  The
// shared expert has a limit of its own and the weight sigmoid(z_shared), where z_shared is the logit
// in column `experts` of the logits' row (`shared_gated`), or 1.
template <typename T, bool WIDE>
__global__ void route_gated_act_kernel(const float* __restrict__ logits, int64_t logits_stride,
                                       const float* __restrict__ correction, const T* proj, int64_t proj_stride,
                                       T* __restrict__ out, int64_t out_stride, float* __restrict__ weights_out,
                                       int experts, int top, int groups, int keep, float route_scale, int ff,
                                       int shared_ff, int shared_gated, float limit, float shared_limit, float alpha) {
    __shared__ float share[ROUTE_MAX_EXPERTS];       // the weight of every expert, 0 if not chosen
    __shared__ float value[ROUTE_MAX_EXPERTS];       // choice scores, -inf once chosen or shut out
    __shared__ float group_score[ROUTE_MAX_EXPERTS];
    __shared__ unsigned char chosen[ROUTE_MAX_EXPERTS];
    __shared__ float shared_weight;
    const int64_t token = blockIdx.x;
    const float* z = logits + token * logits_stride;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z[e])));
        share[e] = s;                                // the plain score for now
        chosen[e] = 0;
        value[e] = correction ? __fadd_rn(s, correction[e]) : s;
    }
    if (threadIdx.x == 0)
        shared_weight = shared_gated ? __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z[experts]))) : 1.0f;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        if (groups > 1 && keep < groups) {
            const int size = experts / groups;
            for (int g = lane; g < groups; g += 32) {
                float first = -INFINITY, second = -INFINITY;
                for (int e = g * size; e < (g + 1) * size; ++e) {
                    const float c = value[e];
                    if (c > first) { second = first; first = c; }
                    else if (c > second) second = c;
                }
                group_score[g] = size > 1 ? __fadd_rn(first, second) : first;
            }
            __syncwarp();
            // the groups that stay are marked +inf, one a round; then every other group is shut out
            for (int round = 0; round < keep; ++round) {
                float best = -INFINITY;
                int where = ROUTE_MAX_EXPERTS;
                for (int g = lane; g < groups; g += 32) {
                    const float c = group_score[g];
                    if (c != INFINITY && (c > best || where == ROUTE_MAX_EXPERTS)) { best = c; where = g; }
                }
#pragma unroll
                for (int delta = 16; delta > 0; delta >>= 1) {
                    const float other = __shfl_xor_sync(0xffffffffu, best, delta);
                    const int other_where = __shfl_xor_sync(0xffffffffu, where, delta);
                    if (other_where < ROUTE_MAX_EXPERTS &&
                        (where == ROUTE_MAX_EXPERTS || other > best || (other == best && other_where < where))) {
                        best = other; where = other_where;
                    }
                }
                if (where >= groups) break;
                if (lane == 0) group_score[where] = INFINITY;
                __syncwarp();
            }
            for (int e = lane; e < experts; e += 32)
                if (group_score[e / size] != INFINITY) value[e] = -INFINITY;
            __syncwarp();
        }
        float sum = 0.0f;
        for (int round = 0; round < top; ++round) {
            float best = -INFINITY;
            int where = ROUTE_MAX_EXPERTS;
            for (int e = lane; e < experts; e += 32)
                if (value[e] > best) { best = value[e]; where = e; }
#pragma unroll
            for (int delta = 16; delta > 0; delta >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, best, delta);
                const int other_where = __shfl_xor_sync(0xffffffffu, where, delta);
                if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
            }
            if (where >= experts) break;                // fewer experts left than `top`
            sum = __fadd_rn(sum, share[where]);
            if (lane == 0) { value[where] = -INFINITY; chosen[where] = 1; }
            __syncwarp();
        }
        const float total = __fadd_rn(sum, 1e-20f);
        for (int e = lane; e < experts; e += 32)
            share[e] = chosen[e] ? __fmul_rn(__fdiv_rn(share[e], total), route_scale) : 0.0f;
    }
    __syncthreads();
    if (weights_out && blockIdx.y == 0)
        for (int e = threadIdx.x; e < experts; e += blockDim.x) weights_out[token * experts + e] = share[e];
    const T* src = proj + token * proj_stride;
    T* dst = out + token * out_stride;
    const int routed = experts * ff;
    int per_block = (routed + shared_ff + gridDim.y - 1) / gridDim.y;
    if (WIDE) per_block = (per_block + 7) / 8 * 8;
    const int begin = blockIdx.y * per_block, end = min(routed + shared_ff, begin + per_block);
    constexpr int STEP = WIDE ? 8 : 1;
    for (int c = begin + threadIdx.x * STEP; c < end; c += blockDim.x * STEP) {
        const bool is_routed = c < routed;
        const int e = is_routed ? c / ff : experts;
        const float weight = is_routed ? share[e] : shared_weight;
        const float lim = is_routed ? limit : shared_limit;
        const int width = is_routed ? ff : shared_ff;
        const int inside = is_routed ? c - e * ff : c - routed;
        const T* gate = src + (is_routed ? (int64_t)e * 2 * ff : (int64_t)2 * routed) + inside;
        const T* up = gate + width;
        float o[STEP];
        if (weight == 0.0f) {
#pragma unroll
            for (int i = 0; i < STEP; ++i) o[i] = 0.0f;
        } else {
            float g[STEP], u[STEP];
            if constexpr (WIDE) {
                unpack_bf16x8(ld_global_16(gate), g);
                unpack_bf16x8(ld_global_16(up), u);
            } else {
                g[0] = to_float<T>(gate[0]);
                u[0] = to_float<T>(up[0]);
            }
#pragma unroll
            for (int i = 0; i < STEP; ++i) {
                const float gg = fminf(g[i], lim);
                const float uu = fminf(fmaxf(u[i], -lim), lim);
                const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__fmul_rn(alpha, gg))));
                o[i] = __fmul_rn(__fmul_rn(__fmul_rn(gg, sig), __fadd_rn(uu, 1.0f)), weight);
            }
        }
        if constexpr (WIDE) *reinterpret_cast<uint4*>(dst + c) = pack_bf16x8(o);
        else dst[c] = from_float<T>(o[0]);
    }
}

// logits float32 [tokens, experts (+ 1 with shared_gated)]; correction float32 [experts] or null; proj
// [tokens, 2 * (experts * ff + shared_ff)] and out [tokens, experts * ff + shared_ff] with row strides;
// weights_out (optional) float32 [tokens, experts].
extern "C" int tvb_route_gated_act(const float* logits, long long logits_stride, const float* correction,
                                   const void* proj, long long proj_stride, void* out, long long out_stride,
                                   float* weights_out, int tokens, int experts, int top, int groups, int keep,
                                   float route_scale, int ff, int shared_ff, int shared_gated, float limit,
                                   float shared_limit, float alpha, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top <= 0 || ff <= 0 || shared_ff < 0 || groups <= 0 ||
        experts % groups || keep <= 0 || keep > groups || (shared_gated && shared_ff == 0))
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const long long columns = (long long)experts * ff + shared_ff;
    const int threads = 256;
    long long split = tokens >= 296 ? 1 : (296 + tokens - 1) / tokens;
    const long long most = (columns + 4 * threads - 1) / (4 * threads);
    if (split > most) split = most;
    if (split > 65535) split = 65535;
    const dim3 grid(tokens, (unsigned)split);
    const bool wide = dtype == TVB_BF16 && ff % 8 == 0 && shared_ff % 8 == 0 && proj_stride % 8 == 0 &&
                      out_stride % 8 == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)out % 16 == 0;
#define GO(T, WIDE) route_gated_act_kernel<T, WIDE><<<grid, threads, 0, s>>>(                                      \
        logits, logits_stride, correction, (const T*)proj, proj_stride, (T*)out, out_stride, weights_out, experts,  \
        top, groups, keep, route_scale, ff, shared_ff, shared_gated, limit, shared_limit, alpha)
    if (dtype == TVB_F32) GO(float, false);
    else if (dtype == TVB_BF16) { if (wide) GO(bf16, true); else GO(bf16, false); }
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}


// ------------------------------------------------------------------------------------------------
// Softmax routing over experts and pass-through slots, with a choice correction, and gated experts.
//
// Per token, from router logits z (float32, one a slot; the first `experts` slots are experts, the last
// `identity` slots hand the layer's input on unchanged and have no tensors): s = softmax(z) over all slots;
// the choice score is s_e + correction_e (`correction` may be null); the `top` slots with the largest choice
// scores are chosen (of equal scores the lower index wins).  A chosen slot's weight is s_e as it is, or, with
// `renormalise`, s_e over the sum of the chosen s.
//
// The packed projection of a token holds [gate_e | up_e] (ff columns each) expert after expert; column c of
// expert e of the output holds act(gate) * up times the expert's weight (exactly 0 if the expert was not
// chosen), act = SiLU.  `identity_out[token]` receives the sum of the chosen pass-through slots' weights: the
// caller adds that many times the layer's input to the result of the down-projection.
template <typename T, bool WIDE>
__global__ void route_softmax_gated_kernel(const float* __restrict__ logits, int64_t logits_stride,
                                           const float* __restrict__ correction, const T* proj, int64_t proj_stride,
                                           T* __restrict__ out, int64_t out_stride, float* __restrict__ weights_out,
                                           float* __restrict__ identity_out, int experts, int identity, int top,
                                           int renormalise, int ff) {
    __shared__ float share[ROUTE_MAX_EXPERTS];       // softmax scores, then the weight of every slot, 0 if not chosen
    __shared__ float value[ROUTE_MAX_EXPERTS];       // choice scores, -inf once chosen
    __shared__ unsigned char chosen[ROUTE_MAX_EXPERTS];
    const int64_t token = blockIdx.x;
    const int slots = experts + identity;
    const float* z = logits + token * logits_stride;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        float top_logit = -INFINITY;
        for (int e = lane; e < slots; e += 32) top_logit = fmaxf(top_logit, z[e]);
#pragma unroll
        for (int delta = 16; delta > 0; delta >>= 1) top_logit = fmaxf(top_logit, __shfl_xor_sync(0xffffffffu, top_logit, delta));
        float total = 0.0f;
        for (int e = lane; e < slots; e += 32) {
            const float w = expf(__fsub_rn(z[e], top_logit));
            share[e] = w;
            total = __fadd_rn(total, w);
        }
        total = warp_sum(total);
        for (int e = lane; e < slots; e += 32) {
            const float s = __fdiv_rn(share[e], total);
            share[e] = s;
            chosen[e] = 0;
            value[e] = correction ? __fadd_rn(s, correction[e]) : s;
        }
        __syncwarp();
        float sum = 0.0f;
        for (int round = 0; round < top; ++round) {
            float best = -INFINITY;
            int where = ROUTE_MAX_EXPERTS;
            for (int e = lane; e < slots; e += 32)
                if (value[e] > best) { best = value[e]; where = e; }
#pragma unroll
            for (int delta = 16; delta > 0; delta >>= 1) {
                const float other = __shfl_xor_sync(0xffffffffu, best, delta);
                const int other_where = __shfl_xor_sync(0xffffffffu, where, delta);
                if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
            }
            if (where >= slots) break;                  // fewer slots than `top`
            sum = __fadd_rn(sum, share[where]);
            if (lane == 0) { value[where] = -INFINITY; chosen[where] = 1; }
            __syncwarp();
        }
        float passed = 0.0f;
        for (int e = lane; e < slots; e += 32) {
            const float w = chosen[e] ? (renormalise ? __fdiv_rn(share[e], sum) : share[e]) : 0.0f;
            share[e] = w;
            if (e >= experts) passed = __fadd_rn(passed, w);
        }
        passed = warp_sum(passed);
        if (lane == 0 && identity_out && blockIdx.y == 0) identity_out[token] = passed;
    }
    __syncthreads();
    if (weights_out && blockIdx.y == 0)
        for (int e = threadIdx.x; e < slots; e += blockDim.x) weights_out[token * slots + e] = share[e];
    const T* src = proj + token * proj_stride;
    T* dst = out + token * out_stride;
    const int routed = experts * ff;
    int per_block = (routed + gridDim.y - 1) / gridDim.y;
    if (WIDE) per_block = (per_block + 7) / 8 * 8;
    const int begin = blockIdx.y * per_block, end = min(routed, begin + per_block);
    constexpr int STEP = WIDE ? 8 : 1;
    for (int c = begin + threadIdx.x * STEP; c < end; c += blockDim.x * STEP) {
        const int e = c / ff;
        const float weight = share[e];
        const T* gate = src + (int64_t)e * 2 * ff + (c - e * ff);
        const T* up = gate + ff;
        float o[STEP];
        if (weight == 0.0f) {
#pragma unroll
            for (int i = 0; i < STEP; ++i) o[i] = 0.0f;
        } else {
            float g[STEP], u[STEP];
            if constexpr (WIDE) {
                unpack_bf16x8(ld_global_16(gate), g);
                unpack_bf16x8(ld_global_16(up), u);
            } else {
                g[0] = to_float<T>(gate[0]);
                u[0] = to_float<T>(up[0]);
            }
#pragma unroll
            for (int i = 0; i < STEP; ++i)
                o[i] = __fmul_rn(__fmul_rn(__fdiv_rn(g[i], __fadd_rn(1.0f, expf(-g[i]))), u[i]), weight);
        }
        if constexpr (WIDE) *reinterpret_cast<uint4*>(dst + c) = pack_bf16x8(o);
        else dst[c] = from_float<T>(o[0]);
    }
}

// logits float32 [tokens, experts + identity]; correction float32 [experts + identity] or null; proj
// [tokens, 2 * experts * ff] and out [tokens, experts * ff] with row strides; weights_out (optional) float32
// [tokens, experts + identity]; identity_out (needed with identity > 0) float32 [tokens].
extern "C" int tvb_route_softmax_gated(const float* logits, long long logits_stride, const float* correction,
                                       const void* proj, long long proj_stride, void* out, long long out_stride,
                                       float* weights_out, float* identity_out, int tokens, int experts, int identity,
                                       int top, int renormalise, int ff, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || identity < 0 || experts + identity > ROUTE_MAX_EXPERTS || top <= 0 || ff <= 0 ||
        (identity > 0 && !identity_out))
        return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const long long columns = (long long)experts * ff;
    const int threads = 256;
    long long split = tokens >= 296 ? 1 : (296 + tokens - 1) / tokens;
    const long long most = (columns + 4 * threads - 1) / (4 * threads);
    if (split > most) split = most;
    if (split > 65535) split = 65535;
    const dim3 grid(tokens, (unsigned)split);
    const bool wide = dtype == TVB_BF16 && ff % 8 == 0 && proj_stride % 8 == 0 && out_stride % 8 == 0 &&
                      (uintptr_t)proj % 16 == 0 && (uintptr_t)out % 16 == 0;
#define GO(T, WIDE) route_softmax_gated_kernel<T, WIDE><<<grid, threads, 0, s>>>(                                  \
        logits, logits_stride, correction, (const T*)proj, proj_stride, (T*)out, out_stride, weights_out,          \
        identity_out, experts, identity, top, renormalise, ff)
    if (dtype == TVB_F32) GO(float, false);
    else if (dtype == TVB_BF16) { if (wide) GO(bf16, true); else GO(bf16, false); }
    else return TVB_BAD_ARGUMENT;
#undef GO
    return tvb_last_error();
}
