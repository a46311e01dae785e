// Kernels of latent attention (keys and values that are up-projections of a cached low-rank latent):
//
//  * latent_kv_store: the row a token leaves in the cache.  From the down projection x [T, R + r] (float32):
//    the first R entries divided by their root mean square (eps inside the root) and multiplied by a weight
//    are the latent; the last r entries are the key part that carries the position and is shared by all
//    heads: its first `rot_dims` entries are rotated (entry i paired with i + rot_dims / 2, angle
//    position * inv_freq[i]), the others pass.  Norm, angles and rotation in float32, one rounding at the
//    store into the paged plane [slots, R + r].  The same launch can norm the query latent of the token, which
//    is another column block of the same down projection.
//  * rotate_slice: the same rotation for a slice of `width` entries of every head of a [T, nh, ...] tensor,
//    written to a slice of another tensor (the queries' rotated part, next to their absorbed part).
//  * rms_rows: x / sqrt(mean(x^2) + eps) * weight for rows of a float32 matrix with a row stride of its own
//    (a column block of a fused projection's output), stored in the compute dtype.
#include "common.cuh"

namespace prism {

template <typename T>
__global__ void latent_kv_store_kernel(const float* __restrict__ x_in, long long x_stride,
                                       const void* __restrict__ weight, int weight_bf16, float eps, int R, int r,
                                       int rot_dims, const float* __restrict__ inv_freq, T* __restrict__ cache,
                                       const int* __restrict__ block_table, int bt_width,
                                       const int* __restrict__ positions, const int* __restrict__ tok_seg,
                                       int page_size, int num_pages, int max_pos, int* err,
                                       const float* __restrict__ xq_in, int q_rank, const void* __restrict__ q_weight,
                                       int q_weight_bf16, T* __restrict__ q_out, long long q_out_stride) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    if (q_out != nullptr) {         // the query latent of the same token (same row stride), normed, in the same launch
        const float* xq = pdl_fresh(xq_in) + (size_t)blockIdx.x * x_stride;
        float sq = 0.f;
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) sq += xq[c] * xq[c];
        sq = block_sum(sq, scratch);
        const float invq = 1.f / sqrtf(sq / (float)q_rank + eps);
        T* o = q_out + (size_t)blockIdx.x * q_out_stride;
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
            o[c] = from_float<T>(xq[c] * invq * load_param(q_weight, q_weight_bf16, c));
    }
    const float* x = pdl_fresh(x_in) + (size_t)blockIdx.x * x_stride;
    const int pos = positions[blockIdx.x];
    float ss = 0.f;
    for (int c = threadIdx.x; c < R; c += blockDim.x) ss += x[c] * x[c];
    ss = block_sum(ss, scratch);
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_POSITION_RANGE);
        return;
    }
    const int page = block_table[(size_t)tok_seg[blockIdx.x] * bt_width + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_PAGE_RANGE);
        return;
    }
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * (size_t)(R + r);
    const float inv = 1.f / sqrtf(ss / (float)R + eps);
    for (int c = threadIdx.x; c < R; c += blockDim.x) dst[c] = from_float<T>(x[c] * inv * load_param(weight, weight_bf16, c));
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float u = x[R + i], v = x[R + i + half];
        dst[R + i] = from_float<T>(u * cs - v * sn);
        dst[R + i + half] = from_float<T>(v * cs + u * sn);
    }
    for (int c = rot_dims + threadIdx.x; c < r; c += blockDim.x) dst[R + c] = from_float<T>(x[R + c]);
}

// one warp per (token, head)
template <typename T>
__global__ void rotate_slice_kernel(const T* __restrict__ in_, long long in_tok_stride, int in_head_stride,
                                    T* __restrict__ out, long long out_tok_stride, int out_head_stride, int width,
                                    int rot_dims, const float* __restrict__ inv_freq,
                                    const int* __restrict__ positions, int Ttot, int nh) {
    pdl_trigger();
    pdl_wait();
    const T* in = pdl_fresh(in_);
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)Ttot * nh) return;
    const int t = (int)(w / nh), h = (int)(w % nh);
    const T* src = in + (size_t)t * in_tok_stride + (size_t)h * in_head_stride;
    T* dst = out + (size_t)t * out_tok_stride + (size_t)h * out_head_stride;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    for (int i = lane; i < half; i += 32) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float u = to_float(src[i]), v = to_float(src[i + half]);
        dst[i] = from_float<T>(u * cs - v * sn);
        dst[i + half] = from_float<T>(v * cs + u * sn);
    }
    for (int c = rot_dims + lane; c < width; c += 32) dst[c] = src[c];
}

template <typename T>
__global__ void rms_rows_kernel(const float* __restrict__ x_in, long long x_stride, const void* __restrict__ weight,
                                int weight_bf16, float eps, T* __restrict__ out, long long out_stride, int width) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const float* x = pdl_fresh(x_in) + (size_t)blockIdx.x * x_stride;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss += x[c] * x[c];
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)width + eps);
    T* o = out + (size_t)blockIdx.x * out_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        o[c] = from_float<T>(x[c] * inv * load_param(weight, weight_bf16, c));
}

}  // namespace prism

PRISM_EXPORT int prism_rms_rows(const float* x, long long x_stride, const void* weight, int weight_dtype, float eps,
                                void* out, long long out_stride, int dtype, int rows, int width, cudaStream_t stream) {
    if (rows <= 0 || width <= 0) return 0;
    const int wb = weight_dtype == PRISM_DTYPE_BF16;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::rms_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x,
                                         x_stride, weight, wb, eps, (__nv_bfloat16*)out, out_stride, width);
    return (int)prism::launch_kernel(prism::rms_rows_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, x_stride,
                                     weight, wb, eps, (float*)out, out_stride, width);
}

// x: float32 [T, R + r] with row stride x_stride; cache: plane [slots, R + r] of `dtype`.  xq (null: none):
// float32 [T, q_rank] with the same row stride (another column block of the same product), RMS-normed with
// q_weight into q_out [T, q_rank] of `dtype` by the same launch.
PRISM_EXPORT int prism_latent_kv_store(const float* x, long long x_stride, const void* weight, int weight_dtype,
                                       float eps, int R, int r, int rot_dims, const float* inv_freq, void* cache,
                                       int dtype, const int* block_table, int bt_width, const int* positions,
                                       const int* tok_seg, int T, int page_size, int num_pages, int max_pos, int* err,
                                       const float* xq, int q_rank, const void* q_weight, int q_weight_dtype,
                                       void* q_out, long long q_out_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (R <= 0 || r < 0 || rot_dims < 0 || rot_dims > r || rot_dims % 2) return (int)cudaErrorInvalidValue;
    if (q_out != nullptr && (xq == nullptr || q_weight == nullptr || q_rank <= 0)) return (int)cudaErrorInvalidValue;
    const int wb = weight_dtype == PRISM_DTYPE_BF16, qwb = q_weight_dtype == PRISM_DTYPE_BF16;
    const int threads = R >= 1024 ? 256 : 128;
    if (dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::latent_kv_store_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, x,
                                         x_stride, weight, wb, eps, R, r, rot_dims, inv_freq, (__nv_bfloat16*)cache,
                                         block_table, bt_width, positions, tok_seg, page_size, num_pages, max_pos, err, xq,
                                         q_rank, q_weight, qwb, (__nv_bfloat16*)q_out, q_out_stride);
    return (int)prism::launch_kernel(prism::latent_kv_store_kernel<float>, dim3(T), dim3(threads), 0, stream, x, x_stride,
                                     weight, wb, eps, R, r, rot_dims, inv_freq, (float*)cache, block_table, bt_width,
                                     positions, tok_seg, page_size, num_pages, max_pos, err, xq, q_rank, q_weight, qwb,
                                     (float*)q_out, q_out_stride);
}

// in/out point at the slice's first entry of head 0 of token 0; strides in elements.
PRISM_EXPORT int prism_rotate_slice(const void* in, long long in_tok_stride, int in_head_stride, void* out,
                                    long long out_tok_stride, int out_head_stride, int dtype, int width, int rot_dims,
                                    const float* inv_freq, const int* positions, int T, int nh, cudaStream_t stream) {
    if (T <= 0 || nh <= 0 || width <= 0) return 0;
    if (rot_dims < 0 || rot_dims > width || rot_dims % 2) return (int)cudaErrorInvalidValue;
    const int warps = 4;
    const long long total = (long long)T * nh;
    const int blocks = (int)((total + warps - 1) / warps);
    if (dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::rotate_slice_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, stream,
                                         (const __nv_bfloat16*)in, in_tok_stride, in_head_stride, (__nv_bfloat16*)out,
                                         out_tok_stride, out_head_stride, width, rot_dims, inv_freq, positions, T, nh);
    return (int)prism::launch_kernel(prism::rotate_slice_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream,
                                     (const float*)in, in_tok_stride, in_head_stride, (float*)out, out_tok_stride,
                                     out_head_stride, width, rot_dims, inv_freq, positions, T, nh);
}
