// Store of a step's new rows into a paged cache plane [slots, width]: the row of the token at position p of
// request seg goes to slot block_table[seg][p / page_size] * page_size + p % page_size.  For layers whose
// keys and values differ in size (each plane gets its own call) or are not rotated.  A page id outside the
// pool or a position outside [0, max_pos) is reported and the row skipped.
#include "common.cuh"
#include "vec.cuh"

namespace prism {

template <typename T>
__global__ void cache_store_kernel(const T* __restrict__ src_in, long long src_stride, T* __restrict__ cache, int width,
                                   const int* __restrict__ block_table, int bt_width,
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
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * width;
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

}  // namespace prism

PRISM_EXPORT int prism_cache_store(const void* src, long long src_stride, void* cache, int dtype, int width,
                                   const int* block_table, int bt_width, const int* positions, const int* tok_seg,
                                   int T, int page_size, int num_pages, int max_pos, int* err, cudaStream_t stream) {
    if (T <= 0 || width <= 0) return 0;
    const int threads = width >= 2048 ? 256 : 128;
    if (dtype == PRISM_DTYPE_BF16) {
        const int vec = width % 8 == 0 && src_stride % 8 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)cache % 16 == 0;
        return (int)prism::launch_kernel(prism::cache_store_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                                         (const __nv_bfloat16*)src, src_stride, (__nv_bfloat16*)cache, width, block_table,
                                         bt_width, positions, tok_seg, page_size, num_pages, max_pos, vec, err);
    }
    const int vec = width % 8 == 0 && src_stride % 8 == 0 && (uintptr_t)src % 32 == 0 && (uintptr_t)cache % 32 == 0;
    return (int)prism::launch_kernel(prism::cache_store_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)src,
                                     src_stride, (float*)cache, width, block_table, bt_width, positions, tok_seg, page_size,
                                     num_pages, max_pos, vec, err);
}
