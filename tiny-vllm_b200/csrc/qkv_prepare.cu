// From a packed projection row to prepared queries and cached keys and values, for attention
// mixers whose sizes and steps are all parameters.  One warp per (token, head).
//
//   q heads   [optional RMS norm over the head, with or without a weight] -> [optional rotation]
//             -> written back where they stand
//   k heads   the same, then written to the key cache at the token's slot
//   v heads   [optional blend (1 - l) v + l v_first with a scalar l read from the device]
//             -> written to the value cache
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

template <typename T, typename W>
__global__ void qkv_prepare_kernel(
    T* proj, int64_t token_stride, int q_at, int k_at, int v_at, int num_q, int num_kv, int key_dim,
    int value_dim, int norm_mode, const W* __restrict__ q_weight, const W* __restrict__ k_weight, float eps,
    const float* __restrict__ inv_freq, int rot_dims, int pairing, const int* __restrict__ positions,
    const int* __restrict__ slots, T* __restrict__ key_cache, T* __restrict__ value_cache, int page_size,
    const T* v_first, int64_t v_first_stride, const T* __restrict__ blend, int tokens) {
    const int heads = num_q + 2 * num_kv;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (int64_t)tokens * heads) return;
    const int lane = threadIdx.x & 31;
    const int token = (int)(row / heads), head = (int)(row % heads);
    T* token_row = proj + (int64_t)token * token_stride;
    const int slot = slots ? slots[token] : -1;

    if (head >= num_q + num_kv) {                       // a value head
        if (slot < 0) return;
        const int g = head - num_q - num_kv;
        const T* src = token_row + v_at + (int64_t)g * value_dim;
        T* dst = value_cache + (((int64_t)(slot / page_size) * num_kv + g) * page_size + slot % page_size) * value_dim;
        if (v_first) {
            const float l = to_float<T>(blend[0]);
            const float keep = __fsub_rn(1.0f, l);
            const T* first = v_first + (int64_t)token * v_first_stride + (int64_t)g * value_dim;
            for (int i = lane; i < value_dim; i += 32)
                dst[i] = from_float<T>(__fadd_rn(__fmul_rn(keep, to_float<T>(src[i])),
                                                 __fmul_rn(l, to_float<T>(first[i]))));
        } else {
            for (int i = lane; i < value_dim; i += 32) dst[i] = src[i];
        }
        return;
    }
    const bool is_key = head >= num_q;
    if (is_key && slot < 0) return;
    T* src = is_key ? token_row + k_at + (int64_t)(head - num_q) * key_dim : token_row + q_at + (int64_t)head * key_dim;
    T* dst = is_key ? key_cache + (((int64_t)(slot / page_size) * num_kv + (head - num_q)) * page_size +
                                   slot % page_size) * key_dim
                    : src;
    const W* weight = norm_mode == PREP_NORM_WEIGHT ? (is_key ? k_weight : q_weight) : nullptr;
    const int pairs = key_dim >> 1, turned = inv_freq ? rot_dims >> 1 : 0;

    // pair j of the head: the two dimensions it holds
    int at_a[PREP_MAX_PAIRS], at_b[PREP_MAX_PAIRS];
    float a[PREP_MAX_PAIRS], b[PREP_MAX_PAIRS];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < PREP_MAX_PAIRS; ++i) {
        const int j = lane + 32 * i;
        a[i] = b[i] = 0.0f;
        at_a[i] = at_b[i] = 0;
        if (j < pairs) {
            if (pairing == PREP_PAIR_HALF_SPLIT && j < turned) { at_a[i] = j; at_b[i] = j + turned; }
            else { at_a[i] = 2 * j; at_b[i] = 2 * j + 1; }
            a[i] = to_float<T>(src[at_a[i]]);
            b[i] = to_float<T>(src[at_b[i]]);
            squares = __fadd_rn(squares, __fmaf_rn(a[i], a[i], __fmul_rn(b[i], b[i])));
        }
    }
    if (norm_mode != PREP_NORM_NONE) {
        squares = warp_sum(squares);
        const float inverse_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, (float)key_dim), eps)));
#pragma unroll
        for (int i = 0; i < PREP_MAX_PAIRS; ++i) {
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
    const float position = (float)max(positions[token], 0);
#pragma unroll
    for (int i = 0; i < PREP_MAX_PAIRS; ++i) {
        const int j = lane + 32 * i;
        if (j < pairs) {
            float u = a[i], v = b[i];
            if (j < turned) {
                float s, c;
                sincosf(__fmul_rn(position, inv_freq[j]), &s, &c);
                u = __fsub_rn(__fmul_rn(a[i], c), __fmul_rn(b[i], s));
                v = __fadd_rn(__fmul_rn(b[i], c), __fmul_rn(a[i], s));
            }
            dst[at_a[i]] = from_float<T>(u);
            dst[at_b[i]] = from_float<T>(v);
        }
    }
}

template <typename T, typename W>
static int launch_prepare(void* proj, long long token_stride, int q_at, int k_at, int v_at, int num_q, int num_kv,
                          int key_dim, int value_dim, int norm_mode, const void* qw, const void* kw, float eps,
                          const float* inv_freq, int rot_dims, int pairing, const int* positions, const int* slots,
                          void* key_cache, void* value_cache, int page_size, const void* v_first,
                          long long v_first_stride, const void* blend, int tokens, cudaStream_t s) {
    const int64_t rows = (int64_t)tokens * (num_q + 2 * num_kv);
    const int warps = 4;
    qkv_prepare_kernel<T, W><<<(unsigned)((rows + warps - 1) / warps), warps * 32, 0, s>>>(
        (T*)proj, token_stride, q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim, norm_mode, (const W*)qw,
        (const W*)kw, eps, inv_freq, rot_dims, pairing, positions, slots, (T*)key_cache, (T*)value_cache,
        page_size, (const T*)v_first, v_first_stride, (const T*)blend, tokens);
    return tvb_last_error();
}

extern "C" int tvb_qkv_prepare(void* proj, long long token_stride, int q_at, int k_at, int v_at, int num_q,
                               int num_kv, int key_dim, int value_dim, int norm_mode, const void* q_weight,
                               const void* k_weight, int weight_dtype, float eps, const float* inv_freq,
                               int rot_dims, int pairing, const int* positions, const int* slots,
                               void* key_cache, void* value_cache, int page_size, const void* v_first,
                               long long v_first_stride, const void* blend, int tokens, int dtype, void* stream) {
    if (tokens <= 0) return 0;
    if (key_dim <= 0 || key_dim % 2 || key_dim > 64 * PREP_MAX_PAIRS || value_dim <= 0 || num_q <= 0 || num_kv < 0 ||
        (slots && page_size <= 0) || norm_mode < 0 || norm_mode > 2 ||
        (norm_mode == PREP_NORM_WEIGHT && (!q_weight || !k_weight)) ||
        (inv_freq && (rot_dims <= 0 || rot_dims % 2 || rot_dims > key_dim || pairing < 0 || pairing > 1)) ||
        (v_first && !blend))
        return TVB_BAD_ARGUMENT;
    if ((int64_t)tokens * (num_q + 2 * num_kv) / 4 + 1 > 2147483647LL) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
#define GO(T, W) return launch_prepare<T, W>(proj, token_stride, q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim, \
        norm_mode, q_weight, k_weight, eps, inv_freq, rot_dims, pairing, positions, slots, key_cache, value_cache,    \
        page_size, v_first, v_first_stride, blend, tokens, s)
    if (dtype == TVB_F32 && weight_dtype == TVB_F32) GO(float, float);
    if (dtype == TVB_BF16 && weight_dtype == TVB_BF16) GO(bf16, bf16);
    if (dtype == TVB_BF16 && weight_dtype == TVB_F32) GO(bf16, float);
#undef GO
    return TVB_BAD_ARGUMENT;
}
