// The C interface of the kernel library.  Every function launches on `stream` and returns 0,
// a cudaError_t value, or one of the RB_ERR_* codes of common.cuh; nothing here allocates.
// Element type codes: 0 = float32, 1 = bfloat16.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int rb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H, int vocab,
                 int* status, void* stream);

int rb_add_rmsnorm(float* resid, const float* delta, int n_delta, long long delta_stride, const void* w,
                   int w_dtype, void* out, int out_dtype, const int* rows, int n_rows, int H, float eps,
                   int write_back, void* stream);

int rb_silu_mul(const void* in, int in_dtype, int n_in, long long in_stride, void* out, int out_dtype, int rows,
                int I, int paired, void* stream);

// Keeps the stream busy for about that long (at most a second): the profiler's gate.
int rb_hold(long long microseconds, void* stream);
int rb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream);

int rb_qk_norm_rope_cache(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, void* q_out,
                          int act_dtype, int q_stride, int T, int nq, int nkv, int hd, const void* q_norm_w,
                          const void* k_norm_w, int w_dtype, float eps, const float* inv_freq, int rot_dim,
                          const int* positions, const int* slot_of_token, const int* block_table, int max_pages,
                          void* k_cache, void* v_cache, int write_kv, const void* cos_sin, void* stream);

int rb_rope_table(const int* positions, const float* inv_freq, int T, int half, void* out, void* stream);

int rb_gemm_generic(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias, void* out,
                    int out_dtype, int M, int N, int K, long long ldx, long long ldo, int splits,
                    long long split_stride, void* stream);

// The limit, in clock cycles, of every barrier wait in the tensor-core products (cycles <= 0: the default,
// about two seconds), and a switch for tests of the give-up path: while it is set a few-token product
// never requests its first K block, so the warp that waits for it runs into the limit, records
// RB_ERR_TIMEOUT in the status word and the block unwinds.
void rb_gemm_tcgen05_set_wait(long long cycles, int withhold_first_stage);
int rb_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int out_dtype, int M, int N,
                    int K, long long ldx, long long ldo, int splits, long long split_stride, int stages,
                    int gated, int* status, void* stream);

int rb_gemm_tcgen05_gated_pair(const void* x, const void* w, const float* bias, void* h, int M, int N, int K,
                               long long ldx, long long ldh, const float* row_sumsq, int row_groups,
                               long long row_sumsq_ld, float row_eps, int stages, int* status, void* stream);

int rb_gemm_tcgen05_residual(const void* x, const void* w, const float* bias, int M, int N, int K, long long ldx,
                             int splits, float* resid, long long ld_resid, const void* next_w, int next_w_f32,
                             void* xhat, long long ld_xhat, float* sumsq, long long ld_sumsq, int stages,
                             int* status, void* stream);

int rb_gemm_tcgen05_qkv_rope(const void* x, const void* w, const float* bias, int M, int N, int K, long long ldx,
                             void* q_out, long long q_ld, void* k_cache, void* v_cache, const int* positions,
                             const int* slot_of_token, const int* block_table, int max_pages, const void* q_norm_w,
                             const void* k_norm_w, int norm_w_f32, float norm_eps, const float* cos_sin, int nq,
                             int nkv, int stages, int* status, void* stream);

int rb_gemm_tcgen05_add(const void* x, const void* w, const float* bias, float* resid, int M, int N, int K,
                        long long ldx, long long ld_resid, int stages, int* status, void* stream);

int rb_attention_generic(const void* q, int q_stride, void* out, int o_stride, int dtype, const void* k_cache,
                         const void* v_cache, const int* block_table, int max_pages, const int* seq_slot,
                         const int* cu_q, const int* kv_len, int B, int max_q_len, int nq, int nkv, int hd,
                         float scale, int window, int chunk, int n_chunks, float* part_acc, float* part_ml,
                         void* stream);

int rb_attention_prefill(const void* q, int q_stride, void* out, int o_stride, const void* k_cache,
                         const void* v_cache, const int* block_table, int max_pages, const int* seq_slot,
                         const int* cu_q, const int* kv_len, int B, int max_q_len, int nq, int nkv, int hd, float scale,
                         int window, void* stream);

int rb_attention_prefill_tc5(const void* q, int q_stride, int T, void* out, int o_stride, const void* k_cache,
                             const void* v_cache, int n_pages, const int* block_table, int max_pages,
                             const int* seq_slot, const int* cu_q, const int* kv_len, int B, int max_q_len, int nq,
                             int nkv, int hd, float scale, int window, int heads_first, int* status, void* stream);

int rb_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                        const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window, int n_chunks,
                        int pages_per_block, float* part_acc, float* part_ml, int* counters, void* out, int o_stride,
                        void* stream);

int rb_attention_decode_fused(const float* proj, int n_in, long long in_stride, int row_stride, const void* q_norm_w,
                              const void* k_norm_w, int w_f32, float eps, const float* cos_sin, int write_kv,
                              const float* row_sumsq, int row_groups, long long row_sumsq_ld, float row_eps,
                              int row_width, void* k_cache, void* v_cache, const int* block_table, int max_pages, const int* seq_slot,
                              const int* cu_q, const int* kv_len, int B, int nq, int nkv, int hd, float scale,
                              int window, int n_chunks, int pages_per_block, float* part_acc, float* part_ml,
                              int* counters, void* out, int o_stride, void* stream);

int rb_attention_merge(const float* part_acc, const float* part_ml, void* out, int o_stride, int dtype,
                       const int* positions, const int* slot_of_token, int T, int nq, int hd, int chunk,
                       int n_chunks, int window, void* stream);

int rb_argmax(const float* logits, long long row_stride, int rows, int V, int* out, float* scratch_v,
              int* scratch_i, int slices, void* stream);

int rb_sample(float* logits, long long row_stride, int n, int V, const void* rows, const int* history, int* out,
              void* stream);

// Reader of safetensors files (safetensors_reader.cu): open and check the header, list the tensors, copy one
// tensor's bytes to host or device memory, close.
void* rb_st_open(const char* path, char* err, int err_len);
int rb_st_count(const void* handle);
int rb_st_entry(const void* handle, int i, const char** name, const char** dtype, int* rank, long long* shape,
                long long* nbytes);
int rb_st_metadata_count(const void* handle);
int rb_st_metadata(const void* handle, int i, const char** key, const char** value);
int rb_st_read(void* handle, int i, void* dst, long long dst_bytes, int on_device, void* stream);
void rb_st_close(void* handle);

#ifdef __cplusplus
}
#endif
