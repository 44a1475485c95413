// Internal interface between the C ABI (fsvd_api.cu) and the tiled tensor-core path for batches of
// 9..128 sequences (fsvd_tile.cu).  Not part of the public header.
#pragma once
#include <stddef.h>

struct fsvd_dims;
struct fsvd_layer;
struct fsvd_tile_model;
struct fsvd_exchange;

// provided by fsvd_api.cu: the library's last-error text and launch counter
void fsvd_tile_set_error(int code, const char* msg);
void fsvd_tile_count_launch();
void fsvd_tile_count_launches(long long n);
long long fsvd_tile_launches();

// provided by fsvd_tile.cu
size_t fsvd_tile_workspace_bytes(const fsvd_dims* dims);
int fsvd_tile_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab, const void* sin_tab,
                           const int* cache_seqlens, const void* x_in, void* x_out, void* ws, size_t ws_bytes,
                           long long wait_limit, void* stream);
int fsvd_tile_tp_decode_layer(const fsvd_dims* dims, const fsvd_layer* layer, const void* cos_tab, const void* sin_tab,
                              const int* cache_seqlens, const void* x_in, const void* x_norm_in, void* x_out,
                              const void* next_norm_w, void* x_norm_out, fsvd_exchange* ex, void* ws, size_t ws_bytes,
                              long long wait_limit, void* stream);
int fsvd_tile_model_create(const fsvd_dims* dims, const fsvd_layer* layers, const void* embed, const void* final_norm_w,
                           const void* lm_head, const void* cos_tab, const void* sin_tab, int max_steps, long long wait_limit,
                           fsvd_tile_model** out);
int fsvd_tile_model_destroy(fsvd_tile_model* m);
int fsvd_tile_model_step(fsvd_tile_model* m, int n_steps, void* stream);
void fsvd_tile_model_buffers(fsvd_tile_model* m, int** tokens, int** seqlens, int** token_log, int** step_counter,
                             float** logits, float** hidden);
void* fsvd_tile_model_ws(fsvd_tile_model* m);
int fsvd_tile_model_launches_per_step(fsvd_tile_model* m);
int fsvd_tile_model_reset(fsvd_tile_model* m, void* stream);
