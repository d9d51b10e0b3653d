// Routing of a mixture of experts and the experts' activation in one pass.
//
// Per token: the `top` experts with the largest router logits (float32; of equal logits the lower
// index wins) get the softmax over their logits alone as weights, all others weight 0.  Then the
// packed up-projection [experts * ff | shared_ff] of the token becomes the input of the packed
// down-projection: column c of expert e holds act(up[c]) * weight_e (exactly 0 for an expert that
// was not chosen), the shared expert's columns hold act(up[c]); act is relu(z)^2 or SiLU.  The
// down-projection over all columns at once is then the weighted sum of the chosen experts' outputs
// plus the shared expert's.  Weights and activation are float32, one rounding to the storage type.
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
