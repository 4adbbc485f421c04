// Operations on the float32 residual stream and the logits that the pre-norm blocks with a
// layer scale use: an embedding lookup with a constant factor, the residual sum under a
// per-feature scale fused with the norm that follows (layer norm or RMS norm), and the soft
// cap of the logits. All arithmetic is float32.
#include "common.cuh"

namespace mb {

// out[t, :] = table[ids[t], :] * scale, written into the float32 residual stream.
__global__ void embed_scaled_kernel(const int* __restrict__ ids, const void* __restrict__ table,
                                    int table_dtype, float scale, float* __restrict__ out,
                                    int hidden, int vocab) {
    grid_dependency_sync();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
#ifdef MB_BOUNDS_CHECK
    if (!ok && threadIdx.x == 0) check_report(MB_CHECK_TOKEN, id, vocab);
#endif
    const int64_t base = (int64_t)(ok ? id : 0) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[(int64_t)t * hidden + c] = ok ? load_as_float(table, base + c, table_dtype) * scale : 0.f;
}

// h <- h + delta * scale (delta and scale optional; scale one number per feature), then, when
// a norm weight is given, out = (x - mean) / sqrt(var + eps) * w of the new row (center = 1;
// var is the mean of the squared deviations) or x / sqrt(mean(x^2) + eps) * w (center = 0).
// With `rows` only the rows listed are normalised (out row r from stream row rows[r]) and
// the stream is left as it was. One block per row; the row stays in shared memory between
// the sums, so mean and variance are taken in two passes over the same numbers.
template <typename TD, typename TO>
__global__ void scaled_add_norm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const void* __restrict__ scale, int scale_dtype,
                                       const void* __restrict__ w, int w_dtype, float eps,
                                       int center, TO* __restrict__ out,
                                       const int* __restrict__ rows, int hidden) {
    grid_dependency_sync();
    extern __shared__ float row_s[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = (int64_t)(rows ? rows[r] : r) * hidden;
    const int64_t dst = (int64_t)r * hidden;
    float sum = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float x = h[src + c];
        if (delta) {
            const float s = scale ? load_as_float(scale, c, scale_dtype) : 1.f;
            x = fmaf(to_float(delta[src + c]), s, x);
            if (!rows) h[src + c] = x;
        }
        row_s[c] = x;
        sum += x;
    }
    if (w == nullptr) return;
    float mean = 0.f;
    if (center) mean = block_sum(sum, scratch) / (float)hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float d = row_s[c] - mean;
        ss += d * d;
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[dst + c] = from_float<TO>((row_s[c] - mean) * rstd * load_as_float(w, c, w_dtype));
}

// x <- cap * tanh(x / cap)
__global__ void softcap_kernel(float* __restrict__ x, int64_t total, float cap) {
    grid_dependency_sync();
    const float inv = 1.f / cap;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_embed_scaled(const int* ids, const void* table, int table_dtype, float scale,
                              float* out, int tokens, int hidden, int vocab, void* stream) {
    if (tokens <= 0) return MB_OK;
    MB_LAUNCH((embed_scaled_kernel), tokens, 256, 0, (cudaStream_t)stream, ids, table, table_dtype,
              scale, out, hidden, vocab);
    return launch_status();
}

// delta_dtype / out_dtype: MB_F32 or MB_BF16. delta, scale, w, out and rows may each be null
// (w null: only the sum is made; out is then not touched).
MB_EXPORT int mb_scaled_add_norm(float* h, const void* delta, int delta_dtype, const void* scale,
                                 int scale_dtype, const void* w, int w_dtype, float eps, int center,
                                 void* out, int out_dtype, const int* rows, int count, int hidden,
                                 void* stream) {
    if (count <= 0 || hidden <= 0) return MB_OK;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 160 * 1024) return MB_ERR_UNSUPPORTED_SIZE;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define MB_SAN_CASE(TD, TO)                                                                       \
    do {                                                                                          \
        static size_t raised = 0;                                                                 \
        if (smem > 48 * 1024 && smem > raised) {                                                  \
            if (cudaFuncSetAttribute(scaled_add_norm_kernel<TD, TO>,                              \
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=   \
                cudaSuccess)                                                                      \
                return MB_ERR_UNSUPPORTED_SIZE;                                                   \
            raised = smem;                                                                        \
        }                                                                                         \
        MB_LAUNCH((scaled_add_norm_kernel<TD, TO>), count, threads, smem, s, h, (const TD*)delta, \
                  scale, scale_dtype, w, w_dtype, eps, center, (TO*)out, rows, hidden);           \
    } while (0)
    if (delta_dtype == MB_F32 && out_dtype == MB_F32) MB_SAN_CASE(float, float);
    else if (delta_dtype == MB_F32 && out_dtype == MB_BF16) MB_SAN_CASE(float, bf);
    else if (delta_dtype == MB_BF16 && out_dtype == MB_F32) MB_SAN_CASE(bf, float);
    else if (delta_dtype == MB_BF16 && out_dtype == MB_BF16) MB_SAN_CASE(bf, bf);
    else return MB_ERR_BAD_DTYPE;
#undef MB_SAN_CASE
    return launch_status();
}

MB_EXPORT int mb_softcap(float* x, long long total, float cap, void* stream) {
    if (total <= 0) return MB_OK;
    if (!(cap > 0.f)) return MB_ERR_UNSUPPORTED_SIZE;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    MB_LAUNCH((softcap_kernel), blocks, 256, 0, (cudaStream_t)stream, x, (int64_t)total, cap);
    return launch_status();
}
