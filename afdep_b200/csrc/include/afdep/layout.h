// Geometry of one Buffer: the wire record, and where every array lives inside a rank's
// symmetric heap.  Plain C++ shared by host and device code; every rank derives the same
// numbers from the same Config, so no offsets are ever exchanged.
//
// Differences from the reference's layout (deep_ep/include/deep_ep/common/layout.cuh):
// roles are native, so FFN heaps hold the receive staging and reply rows while attention
// heaps hold only completion flags; there is no fixed 12 MiB workspace sized for 1024 ranks.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define AFDEP_HD __host__ __device__ __forceinline__
#else
#define AFDEP_HD inline
#endif

namespace afdep {

constexpr int kMaxRanks = 8;          // one NVSwitch domain
constexpr int kMaxTopK = 32;
constexpr int kMaxExpertsLocal = 256;
constexpr int kMaxExperts = 2048;

AFDEP_HD size_t align_sz(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Wire record, one per (token, destination FFN rank):
//   [ payload  : hidden * (1 or 2) bytes                ]
//   [ scales   : hidden/128 fp32 (FP8 only), padded to 16 ]
//   [ expert[K] int32 | pos[K] int32 | weight[K] fp32 | src_token int32 ], padded to 16
// expert[k] is the global expert id or -1; pos[k] is the rank of this (token, k) among all
// of the source's choices of that expert, in token order, so the receiver places the row at
//   row_base[source][expert] + pos[k]   without any atomics.
struct Geometry {
    int world, ffn, attn;
    int hidden, top_k, experts_local, num_experts;
    int capacity;       // tokens per attention rank = records per (source, FFN rank) pair
    int fp8;            // payload is e4m3 with fp32 per-128 scales
    int alignment;      // expert segment alignment in rows

    int payload_bytes, scale_bytes, meta_bytes, rec_bytes, row_bytes, scale_groups;
    int meta_off;       // offset of the metadata inside a record

    // FFN-rank heap
    size_t f_cnt;        // uint64 [attn][experts_local + 4]: (epoch << 32 | count) per expert, then records sent
    size_t f_slot_flag;  // uint32 [attn][capacity]
    size_t f_stage;      // records [attn][capacity]
    size_t f_reply;      // bf16 rows [attn][capacity]
    size_t f_bytes;
    // attention-rank heap
    size_t a_reply_flag; // uint32 [ffn][capacity]
    size_t a_bytes;
    // both: barrier words uint32 [world] at offset 0, scratch for primitives after them
    size_t ctrl_bytes;
    size_t aux_off, aux_bytes;   // region for the secondary primitives (send/recv, gather)
};

AFDEP_HD int cnt_stride(const Geometry& g) { return g.experts_local + 4; }

// `scale_packs`: 4-byte scale words per FP8 row.  0 means one fp32 scale per 128 channels; a caller
// whose scales are exponent bytes packed four to a word (UE8M0x4) passes the number of words.  The
// exchange moves the words as they are.
inline Geometry make_geometry(int ffn, int attn, int hidden, int top_k, int num_experts, int capacity, int fp8,
                              int alignment, size_t aux_bytes, int scale_packs = 0) {
    Geometry g{};
    g.world = ffn + attn;
    g.ffn = ffn;
    g.attn = attn;
    g.hidden = hidden;
    g.top_k = top_k;
    g.num_experts = num_experts;
    g.experts_local = num_experts / ffn;
    g.capacity = capacity;
    g.fp8 = fp8;
    g.alignment = alignment;
    g.scale_groups = scale_packs > 0 ? scale_packs : hidden / 128;
    g.payload_bytes = hidden * (fp8 ? 1 : 2);
    g.scale_bytes = fp8 ? (int)align_sz((size_t)g.scale_groups * 4, 16) : 0;
    g.meta_bytes = (int)align_sz((size_t)top_k * 12 + 4, 16);
    g.meta_off = g.payload_bytes + g.scale_bytes;
    g.rec_bytes = (int)align_sz((size_t)g.meta_off + g.meta_bytes, 128);
    g.row_bytes = hidden * 2;
    g.ctrl_bytes = 4096;
    g.aux_off = g.ctrl_bytes;
    g.aux_bytes = align_sz(aux_bytes, 4096);
    size_t base = g.aux_off + g.aux_bytes;

    size_t o = base;
    g.f_cnt = o;
    o = align_sz(o + (size_t)attn * (g.experts_local + 4) * 8, 256);
    g.f_slot_flag = o;
    o = align_sz(o + (size_t)attn * capacity * 4, 256);
    g.f_stage = o;
    o = align_sz(o + (size_t)attn * capacity * g.rec_bytes, 256);
    g.f_reply = o;
    o = align_sz(o + (size_t)attn * capacity * g.row_bytes, 256);
    g.f_bytes = o;

    o = base;
    g.a_reply_flag = o;
    o = align_sz(o + (size_t)ffn * capacity * 4, 256);
    g.a_bytes = o;
    return g;
}

// Status block in mapped pinned host memory: the first kernel that gives up on a wait (or
// meets an illegal route) records why, and the host raises at its next API call.  Nothing
// on the device ever traps.
enum StatusCode : int {
    kOk = 0,
    kTimeoutCounts = 1,      // FFN: a source's count vector never arrived
    kTimeoutRecord = 2,      // FFN: a record's arrival flag never arrived
    kTimeoutReply = 3,       // attention: an FFN rank's reply flag never arrived
    kTimeoutLookback = 4,    // attention: a sibling CTA never published its aggregate
    kTimeoutBarrier = 5,
    kTimeoutAux = 6,         // send/recv, gather or fetch primitive gave up
    kBadRoute = 16,          // id outside [-1, num_experts) or repeated within a token
    kBadIndex = 17,          // bounds check of a computed row/slot failed (debug builds)
};

struct Status {
    int code;        // first error wins; written last, by the thread that claimed the report
    int kernel;      // which kernel reported
    int rank;
    int peer;
    unsigned epoch;
    long long expected;
    long long observed;
    int detail0, detail1;
};

}  // namespace afdep
