// fa_dispatch.cpp — the configuration-label selector of libfa_sm120.so.
//
// goml's dispatcher (libs/fa_sm120/src/fa_dispatch.cpp:14-62) maps a problem
// (batch_heads, seq_len, head_dim, causal, window) to one of eight kernel ids.
// On sm_100a one tcgen05 kernel family serves every cell, so the ids select no
// code here; they are kept as labels with the same mapping because callers and
// the reference's table tests (libs/fa_sm120/test/test_dispatch.c, 29 rows;
// libs/fa_sm120/go/gofa/gofa_test.go:15-37) observe them.  The mapping is
// written as data: exact-match rows first, then range rules, then defaults.
#include <stdio.h>
#include <stdlib.h>

#include "../../include/fa_sm120.h"

namespace {

struct ExactRow {
    int bh, sl, window;  // window: 0 = only when no window, >0 = that window length
    fa_kernel_id_t id;
};

// hd128 cells pinned to a specific label (src/fa_dispatch.cpp:31-55)
const ExactRow kExact128[] = {
    {4, 8192, 1024, FA_KERNEL_V117B}, {4, 4096, 1024, FA_KERNEL_V118}, {8, 8192, 1024, FA_KERNEL_V118},
    {4, 4096, 0, FA_KERNEL_V118},     {16, 2048, 0, FA_KERNEL_V118},   {16, 4096, 0, FA_KERNEL_V96B},
    {32, 2048, 0, FA_KERNEL_V96B},    {128, 2048, 0, FA_KERNEL_V96B},  {64, 4096, 0, FA_KERNEL_V96B},
};

fa_kernel_id_t select_hd128(int bh, int sl, int window) {
    const int w = window > 0 ? window : 0;
    for (const ExactRow& r : kExact128)
        if (r.bh == bh && r.sl == sl && r.window == w) return r.id;
    if (w > 0) return FA_KERNEL_V121;                    // any other windowed cell
    if (bh == 4 && sl <= 2048) return FA_KERNEL_V122;    // small grids
    if (bh == 8 && sl <= 4096) return FA_KERNEL_V118;
    return FA_KERNEL_V121R;                              // everything else
}

fa_kernel_id_t select_hd64(int bh, int sl) {
    const long long tiles = (long long)bh * ((sl + 127) / 128);
    return tiles > 128 ? FA_KERNEL_V89 : FA_KERNEL_V80B;  // src/fa_dispatch.cpp:21-25
}

bool debug_enabled() {
    static int cached = -1;  // FA_SM120_DEBUG=1 traces decisions (src/fa_dispatch.cpp:64-73)
    if (cached < 0) {
        const char* e = getenv("FA_SM120_DEBUG");
        cached = (e && e[0] == '1') ? 1 : 0;
    }
    return cached == 1;
}

}  // namespace

extern "C" fa_kernel_id_t fa_dispatch_select(int bh, int sl, int hd, int causal, int window) {
    fa_kernel_id_t id = FA_KERNEL_NONE;
    if (bh > 0 && sl > 0) {
        if (hd == 128) id = select_hd128(bh, sl, window);
        else if (hd == 64) id = select_hd64(bh, sl);
    }
    if (id != FA_KERNEL_NONE && debug_enabled())
        fprintf(stderr, "[fa_sm120] dispatch bh=%d sl=%d hd=%d causal=%d wnd=%d -> %s\n", bh, sl, hd, causal, window,
                fa_kernel_name(id));
    return id;
}

extern "C" const char* fa_kernel_name(fa_kernel_id_t id) {
    static const struct { fa_kernel_id_t id; const char* name; } names[] = {
        {FA_KERNEL_V121R, "v121r"}, {FA_KERNEL_V121, "v121"}, {FA_KERNEL_V118, "v118"}, {FA_KERNEL_V122, "v122"},
        {FA_KERNEL_V117B, "v117b"}, {FA_KERNEL_V96B, "v96b"}, {FA_KERNEL_V89, "v89"},   {FA_KERNEL_V80B, "v80b"},
    };
    for (const auto& n : names)
        if (n.id == id) return n.name;
    return "<none>";
}
