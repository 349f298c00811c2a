// placeholder: tiled kernels arrive next; the unified entry routes to the coverage kernel
#include "common.cuh"
namespace emlx { int validate_attn(const emlx_attn_args* a, const emlx_pool* pool, bool need_plan); }
extern "C" {
size_t emlx_attn_plan_bytes(int32_t, int32_t, int32_t, int32_t) { return 256; }
size_t emlx_attn_workspace_bytes(int32_t, int32_t, int32_t, int32_t, int32_t) { return 256; }
int emlx_attn_plan(const int32_t*, const int32_t*, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, void*, size_t, void*) { return EMLX_OK; }
int emlx_attn_unified(const emlx_attn_args* a, const emlx_pool* p, void* s) { return emlx_attn_generic(a, p, s); }
int emlx_attn_decode(const emlx_attn_args* a, const emlx_pool* p, void* s) { return emlx_attn_generic(a, p, s); }
int emlx_attn_prefill(const emlx_attn_args* a, const emlx_pool* p, void* s) { return emlx_attn_generic(a, p, s); }
}
