// ref_shim.cu — C entry points around the reference's own CUDA launchers.
//
// TEST INFRASTRUCTURE ONLY. This translation unit is compiled together with the
// reference's kernels/attention.cu (taken from the reference checkout where it lies,
// never copied) into oracle/_ref/libhector_ref_attention.so. That library is the
// unmodified reference implementation of the path: it is used to pin the CPU oracle
// (golden vectors) and as the reference arm of the benchmark. It is never linked
// into, or loaded by, the product library.
//
// The prototypes below restate kernels/kernels.hpp:414-483 of the reference.

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace helios {
namespace kernels {
void launch_kv_cache_update(const half* new_k, const half* new_v, half* k_cache, half* v_cache,
                            int batch_size, int seq_len, int kv_heads, int head_dim,
                            int max_seq_len, int position, cudaStream_t stream);
void launch_kv_cache_update_dp(const half* new_k, const half* new_v, half* k_cache, half* v_cache,
                               int batch_size, int seq_len, int kv_heads, int head_dim,
                               int max_seq_len, const int32_t* d_position, cudaStream_t stream);
void launch_attention_cached_fp16(const half* q, const half* k_cache, const half* v_cache,
                                  half* output, int batch_size, int seq_len, int num_heads,
                                  int num_kv_heads, int head_dim, int max_seq_len, float scale,
                                  int window_size, cudaStream_t stream);
void launch_attention_cached_fp16_dp(const half* q, const half* k_cache, const half* v_cache,
                                     half* output, int batch_size, const int32_t* d_seq_len,
                                     int num_heads, int num_kv_heads, int head_dim,
                                     int max_seq_len, float scale, int window_size,
                                     cudaStream_t stream);
void launch_attention_prefill_cached_fp16(const half* q, const half* k_cache, const half* v_cache,
                                          half* output, int seq_new, int past_len, int num_heads,
                                          int num_kv_heads, int head_dim, int max_seq_len,
                                          float scale, int window_size, cudaStream_t stream);
// kernels/kernels.hpp:331-352
void launch_qk_norm_rope_fp16(half* q, half* k, const half* q_norm_w, const half* k_norm_w, int batch_size,
                              int seq_len, int num_heads, int num_kv_heads, int head_dim, int rotary_dim,
                              int position_offset, float eps, float theta, float scaling_factor,
                              cudaStream_t stream);
void launch_qk_norm_rope_kv_fp16(half* q, half* k, const half* v, const half* q_norm_w, const half* k_norm_w,
                                 half* k_cache, half* v_cache, int batch_size, int seq_len, int num_heads,
                                 int num_kv_heads, int head_dim, int rotary_dim, int position_offset,
                                 const int32_t* d_position_offset, int max_seq_len, float eps, float theta,
                                 float scaling_factor, cudaStream_t stream);
}  // namespace kernels
}  // namespace helios

using namespace helios::kernels;

extern "C" {

int hector_ref_abi_version() { return 2; }

int hector_ref_qk_norm_rope(void* q, void* k, const void* qw, const void* kw, int batch, int seq_len,
                            int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int position,
                            float eps, float theta, float scaling, void* stream) {
    launch_qk_norm_rope_fp16((half*)q, (half*)k, (const half*)qw, (const half*)kw, batch, seq_len, num_heads,
                             num_kv_heads, head_dim, rotary_dim, position, eps, theta, scaling,
                             (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int hector_ref_qk_norm_rope_kv(void* q, void* k, const void* v, const void* qw, const void* kw, void* k_cache,
                               void* v_cache, int batch, int seq_len, int num_heads, int num_kv_heads,
                               int head_dim, int rotary_dim, int position, const int32_t* d_position,
                               int max_seq_len, float eps, float theta, float scaling, void* stream) {
    launch_qk_norm_rope_kv_fp16((half*)q, (half*)k, (const half*)v, (const half*)qw, (const half*)kw,
                                (half*)k_cache, (half*)v_cache, batch, seq_len, num_heads, num_kv_heads,
                                head_dim, rotary_dim, position, d_position, max_seq_len, eps, theta, scaling,
                                (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int hector_ref_kv_cache_update(const void* new_k, const void* new_v, void* k_cache, void* v_cache,
                               int batch, int seq_len, int kv_heads, int head_dim, int max_seq_len,
                               int position, void* stream) {
    launch_kv_cache_update((const half*)new_k, (const half*)new_v, (half*)k_cache, (half*)v_cache,
                           batch, seq_len, kv_heads, head_dim, max_seq_len, position,
                           (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int hector_ref_kv_cache_update_dp(const void* new_k, const void* new_v, void* k_cache,
                                  void* v_cache, int batch, int seq_len, int kv_heads, int head_dim,
                                  int max_seq_len, const int32_t* d_position, void* stream) {
    launch_kv_cache_update_dp((const half*)new_k, (const half*)new_v, (half*)k_cache,
                              (half*)v_cache, batch, seq_len, kv_heads, head_dim, max_seq_len,
                              d_position, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int hector_ref_attention_cached(const void* q, const void* k_cache, const void* v_cache, void* out,
                                int batch, int seq_len, int num_heads, int num_kv_heads,
                                int head_dim, int max_seq_len, float scale, int window_size,
                                void* stream) {
    launch_attention_cached_fp16((const half*)q, (const half*)k_cache, (const half*)v_cache,
                                 (half*)out, batch, seq_len, num_heads, num_kv_heads, head_dim,
                                 max_seq_len, scale, window_size, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int hector_ref_attention_cached_dp(const void* q, const void* k_cache, const void* v_cache,
                                   void* out, int batch, const int32_t* d_seq_len, int num_heads,
                                   int num_kv_heads, int head_dim, int max_seq_len, float scale,
                                   int window_size, void* stream) {
    launch_attention_cached_fp16_dp((const half*)q, (const half*)k_cache, (const half*)v_cache,
                                    (half*)out, batch, d_seq_len, num_heads, num_kv_heads, head_dim,
                                    max_seq_len, scale, window_size, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

int hector_ref_attention_prefill_cached(const void* q, const void* k_cache, const void* v_cache,
                                        void* out, int seq_new, int past_len, int num_heads,
                                        int num_kv_heads, int head_dim, int max_seq_len,
                                        float scale, int window_size, void* stream) {
    launch_attention_prefill_cached_fp16((const half*)q, (const half*)k_cache,
                                         (const half*)v_cache, (half*)out, seq_new, past_len,
                                         num_heads, num_kv_heads, head_dim, max_seq_len, scale,
                                         window_size, (cudaStream_t)stream);
    return (int)cudaGetLastError();
}

}  // extern "C"
