// Folding without the final copyTo: what the background folder keeps in its cache is the folded
// Const::Content itself (logical type, storage element type, splat flag, storage bytes), so that a later
// request can continue from it with further transformations exactly as the reference does
// (utils/constant_folding_in_background.cpp:65-100).
#pragma once

#include "common.h"

namespace vf {

struct Folded {  // a folded content in device memory
    Type type;
    int storage = VF_DT_INVALID;
    bool splat = false;
    void* data = nullptr;  // stream-ordered allocation (cudaMallocAsync); the holder frees it with cudaFreeAsync
    uint64_t nbytes = 0;
};

// ContentAttr::fold over a base in host or device memory, or — with `resume` — the transformations t[0 .. n)
// applied on top of an already folded content. Returns after the result is complete (the context's stream is
// synchronised and its error flags are checked).
Folded fold_keep(vf_ctx* ctx, const vf_content* base, const Folded* resume, const vf_transform* t, int n);

// Content::copyTo of a folded content (arguments as the tail of vf_fold); returns the bytes written.
uint64_t copy_folded(vf_ctx* ctx, const Folded& f, void* dst, uint64_t dst_bytes, int dst_mem_kind, vf_tensor_type* out_type,
                     double* scales_buf, int64_t* zps_buf, int64_t params_cap);

// A device copy of a base content that lives in host memory (complete on return).
void* upload_keep(vf_ctx* ctx, const vf_content& base, uint64_t* nbytes);

}  // namespace vf
