// Internal interface of the per-program specialiser (eltwise_jit.cu).
#pragma once

#include <cuda_runtime.h>

#include <string>

#include "ttlb200.h"

struct ttlb_ctx;
struct ttlb_jit_cache;

bool ttlb_eltwise_jit_available();
std::string ttlb_eltwise_jit_key(const ttlb_eltwise_desc *d);
std::string ttlb_eltwise_jit_source(const ttlb_eltwise_desc *d);
int ttlb_eltwise_jit_launch(ttlb_ctx *ctx, ttlb_jit_cache **cache, const ttlb_eltwise_desc *d, cudaStream_t stream);
void ttlb_jit_cache_destroy(ttlb_jit_cache *c);

// Reductions: `partial` holds partial_floats floats, `partial2` max_groups floats, `counters`
// max_groups + 1 zero-initialised words (the kernel leaves them zero).
std::string ttlb_reduce_jit_key(const ttlb_reduce_desc *r);
std::string ttlb_reduce_jit_source(const ttlb_reduce_desc *r);
int ttlb_reduce_jit_launch(ttlb_ctx *ctx, ttlb_jit_cache **cache, const ttlb_reduce_desc *r, float *partial,
                           size_t partial_floats, float *partial2, unsigned *counters, unsigned max_groups,
                           cudaStream_t stream);

// Row-resident fusion (ttlb_rowfused): reductions over columns + a final element-wise program, one kernel.
std::string ttlb_rowfused_jit_source(const ttlb_rowfused_desc *f);
int ttlb_rowfused_jit_launch(ttlb_ctx *ctx, ttlb_jit_cache **cache, const ttlb_rowfused_desc *f, cudaStream_t stream);
