// Host-side TMA tensor maps shared by the tiled and the prefill kernels.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace emlx {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn();

struct MapPair {
    CUtensorMap k, v;
};
// Maps of the pool (cached per pool address and geometry).
int get_maps(const emlx_pool& pool, MapPair* out);
// Launches the tcgen05 prefill kernel over the plan's 128-row units.  `queue`: two zero-initialised ints of the
// workspace (item counter, finished CTAs).  `wait_late`: the launch right before this one in the stream is the
// short-row kernel of the same attention call; the prefill grid then runs beside it and waits for it at its end.
int launch_prefill(const emlx_attn_args* a, const emlx_pool* pool, const int32_t* plan_class_hdr, const int32_t* unit_seq,
                   const int32_t* unit_row0, const int32_t* unit_tile_lo, const int32_t* unit_cum, const int32_t* unit_order,
                   int32_t* queue, bool wait_late, const MapPair& maps, cudaStream_t stream);
long long* trace_buffer();  // the optional tracing buffer (NULL = off)
bool prefill_supported(int kv_format, int num_q_heads, int num_kv_heads, int head_dim);
// The same without the pool format: head geometry the 128-row kernel can run.
bool prefill_geometry_ok(int num_q_heads, int num_kv_heads, int head_dim);

// 128-row units over an affine pool: scratch behind the attention workspace into which the pages of the sequences
// that own such units are expanded to 16-bit rows (csrc/dequant_pages.cu).
struct DequantScratch {
    int32_t* sbt;      // [S, MB] scratch page table
    uint8_t* q16;      // bf16 queries: fp16 copy of the queries [T, Hq, D] (rows of the sequences served), else nullptr
    uint8_t* out16;    // and the fp16 output rows of the 128-row kernel before they are converted back
    uint8_t* k;        // [cap, 128, Hkv, D] 16-bit
    uint8_t* v;
    int cap;           // pages: max_blocks_per_seq for each sequence the scratch was sized for
};
bool dequant_scratch_layout(const emlx_pool* pool, const emlx_attn_args* a, uint8_t* base, size_t bytes, DequantScratch* out);
int launch_dequant_pages(const emlx_attn_args* a, const emlx_pool* pool, const DequantScratch& sc, cudaStream_t stream);
int launch_convert_out_rows(const emlx_attn_args* a, const emlx_pool* pool, const DequantScratch& sc, cudaStream_t stream);

}  // namespace emlx
