// Store of a step's new rows into one or two paged cache planes [slots, width]: the row of the token at position
// p of request seg goes to slot block_table[seg][p / page_size] * page_size + p % page_size.  For layers whose
// keys and values differ in size (a plane each, of its own width, filled by the same launch) or are not rotated.  A page id outside the
// pool or a position outside [0, max_pos) is reported and the row skipped.
#include "common.cuh"
#include "vec.cuh"

namespace prism {

template <typename T>
__device__ __forceinline__ void copy_row(const T* __restrict__ src, T* __restrict__ dst, int width, int vec) {
    if (vec) {
        for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
            float v[8];
            load8(src + c, v);
            store8(dst + c, v);
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
}

template <typename T>
__global__ void cache_store_kernel(const T* __restrict__ src_in, long long src_stride, T* __restrict__ cache, int width,
                                   const T* __restrict__ src2_in, long long src2_stride, T* __restrict__ cache2, int width2,
                                   int vec2, const int* __restrict__ block_table, int bt_width,
                                   const int* __restrict__ positions, const int* __restrict__ tok_seg,
                                   int page_size, int num_pages, int max_pos, int vec, int* err) {
    pdl_trigger();
    pdl_wait();
    const T* src = pdl_fresh(src_in) + (size_t)blockIdx.x * src_stride;
    const int pos = positions[blockIdx.x];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_POSITION_RANGE);
        return;
    }
    const int page = block_table[(size_t)tok_seg[blockIdx.x] * bt_width + pos / page_size];
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) report_error(err, PRISM_ERR_PAGE_RANGE);
        return;
    }
    const size_t slot = (size_t)page * page_size + pos % page_size;
    copy_row(src, cache + slot * width, width, vec);
    if (cache2 != nullptr)
        copy_row(pdl_fresh(src2_in) + (size_t)blockIdx.x * src2_stride, cache2 + slot * width2, width2, vec2);
}

}  // namespace prism

// src2 / cache2 (null: none): a second plane of width2 entries a slot, filled from rows of its own.
PRISM_EXPORT int prism_cache_store(const void* src, long long src_stride, void* cache, int dtype, int width,
                                   const void* src2, long long src2_stride, void* cache2, int width2,
                                   const int* block_table, int bt_width, const int* positions, const int* tok_seg,
                                   int T, int page_size, int num_pages, int max_pos, int* err, cudaStream_t stream) {
    if (T <= 0 || width <= 0) return 0;
    if (cache2 != nullptr && (src2 == nullptr || width2 <= 0)) return (int)cudaErrorInvalidValue;
    const int threads = width + width2 >= 2048 ? 256 : 128;
    const size_t al = dtype == PRISM_DTYPE_BF16 ? 16 : 32;
    auto vec_ok = [&](const void* s, long long ss, const void* c, int w) {
        return w % 8 == 0 && ss % 8 == 0 && (uintptr_t)s % al == 0 && (uintptr_t)c % al == 0 ? 1 : 0;
    };
    const int vec = vec_ok(src, src_stride, cache, width), vec2 = cache2 != nullptr ? vec_ok(src2, src2_stride, cache2, width2) : 0;
    if (dtype == PRISM_DTYPE_BF16)
        return (int)prism::launch_kernel(prism::cache_store_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                                         (const __nv_bfloat16*)src, src_stride, (__nv_bfloat16*)cache, width,
                                         (const __nv_bfloat16*)src2, src2_stride, (__nv_bfloat16*)cache2, width2, vec2,
                                         block_table, bt_width, positions, tok_seg, page_size, num_pages, max_pos, vec, err);
    return (int)prism::launch_kernel(prism::cache_store_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)src,
                                     src_stride, (float*)cache, width, (const float*)src2, src2_stride, (float*)cache2, width2,
                                     vec2, block_table, bt_width, positions, tok_seg, page_size, num_pages, max_pos, vec, err);
}
