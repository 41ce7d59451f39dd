// Tree broadphase of one env inside its warp: Morton keys of the AABB centres, an in-shared-memory bitonic sort, a
// Karras radix tree, bounds refitted level by level without atomics, and a stackless walk per leaf.  The surviving pairs
// are gathered as one partner bit row per body and written in ascending (a, b) order, which is the canonical order of
// the reference's sorted pair list, so no sort of the output is needed.
// The quantities follow the reference's per-env tree (src/collision/lbvh_batched.cuh:85-135 scene bound + Morton3D30
// keys, :174-216 internal nodes with the index tie-break of lbvh_node.cuh:52-67, :220-241 bound propagation) and its
// walk and filters (src/phi/backend_cuda/ops/broadphase.cu:314-401); the filters are the template's admissibility
// bits (not both static, bitmask / group admitted, not excluded), which do not change from step to step.
#pragma once
#include "nkb_collide.cuh"

namespace nkb {

struct LbvhScratch {
    uint32_t* code;      // P sorted Morton codes
    uint32_t* index;     // P body row of each sorted leaf
    uint32_t* child;     // (B - 1) x 2: child node ids; ids >= B - 1 are leaves (id - (B - 1) = sorted position)
    uint32_t* range;     // (B - 1) x 2: first and last sorted leaf of the node
    float* box;          // (B - 1) x 6
    uint32_t* split_node;// B: internal node whose split lies after sorted leaf k
    uint32_t* ready;     // B: 1 once the node's box is final
    uint32_t* partners;  // B x W bit rows, by body row
};

NKB_DEV LbvhScratch lbvh_bind(const Env& e, uint32_t B) {
    const uint32_t P = lbvh_pow2(B), W = (B + 31u) / 32u, I = B - 1u;
    uint32_t* at = reinterpret_cast<uint32_t*>(e.sm + e.lay->heads);
    LbvhScratch s;
    s.code = at; at += P;
    s.index = at; at += P;
    s.child = at; at += 2u * I;
    s.range = at; at += 2u * I;
    s.box = reinterpret_cast<float*>(at); at += 6u * I;
    s.split_node = at; at += B;
    s.ready = at; at += B;
    at += 2u * B;                       // spare
    s.partners = at;                    // B x W words; lbvh_scratch_words (nkb_types.h) sizes the whole region
    (void)W;
    return s;
}

NKB_DEV uint32_t expand_bits10(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}
NKB_DEV uint32_t morton3d30(float x, float y, float z) {
    x = fminf(fmaxf(x * 1024.0f, 0.0f), 1023.0f);
    y = fminf(fmaxf(y * 1024.0f, 0.0f), 1023.0f);
    z = fminf(fmaxf(z * 1024.0f, 0.0f), 1023.0f);
    return (expand_bits10((uint32_t)x) << 2) | (expand_bits10((uint32_t)y) << 1) | expand_bits10((uint32_t)z);
}
// length of the common prefix of sorted keys i and j; equal codes fall back to the positions, so the tree is valid with
// duplicate codes; -1 outside the range
NKB_DEV int lbvh_delta(const uint32_t* code, int i, int j, int n) {
    if (j < 0 || j >= n) return -1;
    const uint32_t ci = code[i], cj = code[j];
    return ci == cj ? 32 + __clz((uint32_t)(i ^ j)) : __clz(ci ^ cj);
}

// Candidate pairs through the tree, written to the pair list in ascending (a << 16 | b) order.  Returns the pair count.
NKB_DEV uint32_t stage_pairs_lbvh(Env& e) {
    const TemplateView& t = *e.t;
    const uint32_t B = t.B, lane = e.lane;
    const uint32_t cap = t.cfg.max_pairs != 0u && t.cfg.max_pairs < t.cfg.max_contacts ? t.cfg.max_pairs : t.cfg.max_contacts;
    if (B < 2u) return 0u;
    const uint32_t P = lbvh_pow2(B), W = (B + 31u) / 32u, I = B - 1u;
    const LbvhScratch s = lbvh_bind(e, B);
    // ---- scene bound of the box centres (min and max fold exactly in any order) ----
    float mn[3] = {FLT_MAX, FLT_MAX, FLT_MAX}, mx[3] = {-FLT_MAX, -FLT_MAX, -FLT_MAX};
    for (uint32_t b = lane; b < B; b += 32u) {
        const float* a = sm_aabb(e, b);
#pragma unroll
        for (int k = 0; k < 3; ++k) { const float c = 0.5f * (a[k] + a[3 + k]); mn[k] = fminf(mn[k], c); mx[k] = fmaxf(mx[k], c); }
    }
#pragma unroll
    for (int k = 0; k < 3; ++k)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { mn[k] = fminf(mn[k], __shfl_xor_sync(NKB_FULL, mn[k], o)); mx[k] = fmaxf(mx[k], __shfl_xor_sync(NKB_FULL, mx[k], o)); }
    float inv[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) inv[k] = mx[k] > mn[k] ? 1.0f / (mx[k] - mn[k]) : 0.0f;
    for (uint32_t b = lane; b < P; b += 32u) {
        uint32_t code = 0xffffffffu;            // padding sorts to the end
        if (b < B) {
            const float* a = sm_aabb(e, b);
            code = morton3d30((0.5f * (a[0] + a[3]) - mn[0]) * inv[0], (0.5f * (a[1] + a[4]) - mn[1]) * inv[1], (0.5f * (a[2] + a[5]) - mn[2]) * inv[2]);
        }
        s.code[b] = code; s.index[b] = b;
    }
    __syncwarp();
    // ---- bitonic sort of (code, body row): ascending, ties by row, i.e. the order a stable radix sort of the codes gives ----
    for (uint32_t k = 2u; k <= P; k <<= 1u)
        for (uint32_t j = k >> 1u; j > 0u; j >>= 1u) {
            for (uint32_t x = lane; x < P; x += 32u) {
                const uint32_t y = x ^ j;
                if (y > x) {
                    const uint32_t cx = s.code[x], cy = s.code[y], ix = s.index[x], iy = s.index[y];
                    const bool greater = cx > cy || (cx == cy && ix > iy);
                    if (greater == ((x & k) == 0u)) { s.code[x] = cy; s.code[y] = cx; s.index[x] = iy; s.index[y] = ix; }
                }
            }
            __syncwarp();
        }
    // ---- internal nodes (Karras 2012) ----
    const int n = (int)B;
    for (uint32_t i0 = lane; i0 < I; i0 += 32u) {
        const int i = (int)i0;
        const int d = lbvh_delta(s.code, i, i + 1, n) >= lbvh_delta(s.code, i, i - 1, n) ? 1 : -1;
        const int delta_min = lbvh_delta(s.code, i, i - d, n);
        int l_max = 2;
        while (lbvh_delta(s.code, i, i + l_max * d, n) > delta_min) l_max <<= 1;
        int l = 0;
        for (int step = l_max >> 1; step >= 1; step >>= 1)
            if (lbvh_delta(s.code, i, i + (l + step) * d, n) > delta_min) l += step;
        const int j = i + l * d;
        const int delta_node = lbvh_delta(s.code, i, j, n);
        int split = 0, step = l;
        do {
            step = (step + 1) >> 1;
            if (lbvh_delta(s.code, i, i + (split + step) * d, n) > delta_node) split += step;
        } while (step > 1);
        const int gamma = i + split * d + min(d, 0);
        const int first = min(i, j), last = max(i, j);
        s.child[2u * i0] = first == gamma ? I + (uint32_t)gamma : (uint32_t)gamma;
        s.child[2u * i0 + 1u] = last == gamma + 1 ? I + (uint32_t)(gamma + 1) : (uint32_t)(gamma + 1);
        s.range[2u * i0] = (uint32_t)first; s.range[2u * i0 + 1u] = (uint32_t)last;
        s.split_node[gamma] = i0;           // every split position belongs to exactly one internal node
        s.ready[i0] = 0u;
    }
    __syncwarp();
    // ---- bounds: a node merges its children once both are final; passes repeat until the root is (height of the tree) ----
    for (uint32_t pass = 0u; pass < B; ++pass) {
        bool changed = false;
        for (uint32_t i0 = lane; i0 < I; i0 += 32u) {
            if (s.ready[i0] != 0u) continue;
            const uint32_t c0 = s.child[2u * i0], c1 = s.child[2u * i0 + 1u];
            const bool r0 = c0 >= I || s.ready[c0] == 2u, r1 = c1 >= I || s.ready[c1] == 2u;
            if (!(r0 && r1)) continue;
            const float* a = c0 >= I ? sm_aabb(e, s.index[c0 - I]) : s.box + 6u * c0;
            const float* b = c1 >= I ? sm_aabb(e, s.index[c1 - I]) : s.box + 6u * c1;
            float* o = s.box + 6u * i0;
#pragma unroll
            for (int k = 0; k < 3; ++k) { o[k] = fminf(a[k], b[k]); o[3 + k] = fmaxf(a[3 + k], b[3 + k]); }
            s.ready[i0] = 1u;
            changed = true;
        }
        __syncwarp();
        // boxes written in this pass become visible to the next one only: a node never reads a sibling written in the same pass
        for (uint32_t i0 = lane; i0 < I; i0 += 32u) if (s.ready[i0] == 1u) s.ready[i0] = 2u;
        __syncwarp();
        if (!__any_sync(NKB_FULL, changed)) break;
    }
    // ---- walk: lane = sorted leaf; on a miss or after a leaf the walk jumps to the right child of the node whose split lies after
    //      the subtree's last leaf, so no stack is kept ----
    const uint32_t kEnd = 0xffffffffu;
    for (uint32_t k0 = 0u; k0 < B; k0 += 32u) {
        const uint32_t k = k0 + lane;
        if (k < B) {
            const uint32_t a = s.index[k];
            const float* q = sm_aabb(e, a);
            const float q0 = q[0], q1 = q[1], q2 = q[2], q3 = q[3], q4 = q[4], q5 = q[5];
            uint32_t* row = s.partners + a * W;
            for (uint32_t w = 0u; w < W; ++w) row[w] = 0u;
            const uint32_t* adm = t.adm_mask + a * W;
            uint32_t node = 0u;                     // the root
            uint32_t guard = 4u * B;                // a walk visits each node at most once
            while (node != kEnd && guard-- != 0u) {
                const bool leaf = node >= I;
                const uint32_t last = leaf ? node - I : s.range[2u * node + 1u];
                const float* bx = leaf ? sm_aabb(e, s.index[node - I]) : s.box + 6u * node;
                const bool hit = !(q3 < bx[0] || q0 > bx[3] || q4 < bx[1] || q1 > bx[4] || q5 < bx[2] || q2 > bx[5]);
                if (hit && !leaf) { node = s.child[2u * node]; continue; }
                if (hit) {
                    const uint32_t b = s.index[node - I];
                    if (a < b && ((__ldg(adm + (b >> 5)) >> (b & 31u)) & 1u) != 0u) row[b >> 5] |= 1u << (b & 31u);
                }
                node = last + 1u < B ? s.child[2u * s.split_node[last] + 1u] : kEnd;
            }
        }
    }
    __syncwarp();
    // ---- emit: bodies in row order, partners in bit order ----
    uint32_t count = 0u;
    uint32_t* pairs = sm_pairs(e);
    for (uint32_t a0 = 0u; a0 < B; a0 += 32u) {
        const uint32_t a = a0 + lane;
        uint32_t mine = 0u;
        if (a < B) for (uint32_t w = 0u; w < W; ++w) mine += __popc(s.partners[a * W + w]);
        uint32_t scan = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t up = __shfl_up_sync(NKB_FULL, scan, o); if ((int)lane >= o) scan += up; }
        uint32_t at = count + scan - mine;
        if (a < B)
            for (uint32_t w = 0u; w < W; ++w) {
                uint32_t bits = s.partners[a * W + w];
                while (bits != 0u) {
                    const uint32_t b = 32u * w + (uint32_t)__ffs(bits) - 1u;
                    bits &= bits - 1u;
                    if (at < cap) pairs[at] = (a << 16) | b; else e.status |= kStatusPairOverflow;
                    ++at;
                }
            }
        count += __shfl_sync(NKB_FULL, scan, 31);
    }
    __syncwarp();
    return count < cap ? count : cap;
}

}  // namespace nkb
