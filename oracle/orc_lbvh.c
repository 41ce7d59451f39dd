/* Oracle (test infrastructure): the reference's per-env LBVH broadphase, restated serially.
 * Follows src/collision/lbvh_batched.cuh:85-135 (scene bound of the AABB centres, Morton3D30 keys), :265-313 (stable
 * key sort, the job cub::DeviceRadixSort::SortPairs does there), :174-216 (Karras internal nodes on sorted codes with
 * the index tie-break of src/collision/lbvh_node.cuh:52-67), :220-241 (bottom-up bound propagation) and
 * src/phi/backend_cuda/ops/broadphase.cu:314-401 (stack walk emitting i<j, static-static / bitmask / exclusion filters),
 * :476-678 (canonical ascending order of the surviving pairs). */
#include <stdlib.h>

#include "orc.h"
#include "orc_math.h"

typedef struct { int32_t left, right, parent; float lo[3], hi[3]; } lbvh_node;

/* src/collision/morton_codes.cuh */
static uint32_t expand_bits10(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}
static uint32_t morton3d30(float x, float y, float z) {
    x = fminf(fmaxf(x * 1024.0f, 0.0f), 1023.0f);
    y = fminf(fmaxf(y * 1024.0f, 0.0f), 1023.0f);
    z = fminf(fmaxf(z * 1024.0f, 0.0f), 1023.0f);
    return (expand_bits10((uint32_t)x) << 2) | (expand_bits10((uint32_t)y) << 1) | expand_bits10((uint32_t)z);
}
static int clz32(uint32_t v) { return v == 0u ? 32 : __builtin_clz(v); }
/* lbvh_node.cuh:52-67 */
static int lbvh_delta(int i, int j, uint32_t n, const uint32_t *code) {
    if (j < 0 || j >= (int)n) return -1;
    if (code[i] == code[j]) return 32 + clz32((uint32_t)(i ^ j));
    return clz32(code[i] ^ code[j]);
}

/* Builds one env's tree over n leaf boxes.  nodes: 2n - 1 entries, internal nodes first (0 is the root), leaf k of the
 * sorted order at n - 1 + k with its original index in .left.  code/order: n words of scratch each. */
static void lbvh_build(uint32_t n, const float *lo, const float *hi, lbvh_node *nodes, uint32_t *code, uint32_t *order) {
    float mn[3] = {FLT_MAX, FLT_MAX, FLT_MAX}, mx[3] = {-FLT_MAX, -FLT_MAX, -FLT_MAX};
    for (uint32_t i = 0; i < n; ++i)
        for (int k = 0; k < 3; ++k) {
            const float c = 0.5f * (lo[3 * i + k] + hi[3 * i + k]);
            mn[k] = fminf(mn[k], c); mx[k] = fmaxf(mx[k], c);
        }
    float inv[3];
    for (int k = 0; k < 3; ++k) inv[k] = mx[k] > mn[k] ? 1.0f / (mx[k] - mn[k]) : 0.0f;
    uint32_t *raw = (uint32_t *)malloc(sizeof(uint32_t) * n);
    for (uint32_t i = 0; i < n; ++i) {
        float c[3];
        for (int k = 0; k < 3; ++k) c[k] = (0.5f * (lo[3 * i + k] + hi[3 * i + k]) - mn[k]) * inv[k];
        raw[i] = morton3d30(c[0], c[1], c[2]);
        order[i] = i;
    }
    /* stable ascending sort of (code, index): insertion sort keeps equal codes in index order, as a radix sort does */
    for (uint32_t i = 1; i < n; ++i) {
        const uint32_t o = order[i];
        uint32_t j = i;
        while (j > 0 && raw[order[j - 1]] > raw[o]) { order[j] = order[j - 1]; --j; }
        order[j] = o;
    }
    for (uint32_t i = 0; i < n; ++i) code[i] = raw[order[i]];
    free(raw);
    const uint32_t internal = n - 1u;
    for (uint32_t i = 0; i < internal; ++i) nodes[i].parent = -1;
    for (uint32_t k = 0; k < n; ++k) {
        lbvh_node *leaf = nodes + internal + k;
        leaf->left = (int32_t)order[k]; leaf->right = -1; leaf->parent = -1;
        for (int c = 0; c < 3; ++c) { leaf->lo[c] = lo[3 * order[k] + c]; leaf->hi[c] = hi[3 * order[k] + c]; }
    }
    for (int i = 0; i < (int)internal; ++i) {
        const int d_l = lbvh_delta(i, i - 1, n, code), d_r = lbvh_delta(i, i + 1, n, code);
        const int d = d_r >= d_l ? 1 : -1;
        const int delta_min = lbvh_delta(i, i - d, n, code);
        int l_max = 2;
        while (lbvh_delta(i, i + l_max * d, n, code) > delta_min) l_max *= 2;
        int l = 0;
        for (int t = l_max >> 1; t >= 1; t >>= 1)
            if (lbvh_delta(i, i + (l + t) * d, n, code) > delta_min) l += t;
        const int j = i + l * d;
        const int delta_node = lbvh_delta(i, j, n, code);
        int s = 0, t_div = l;
        do {
            t_div = (t_div + 1) >> 1;
            if (lbvh_delta(i, i + (s + t_div) * d, n, code) > delta_node) s += t_div;
        } while (t_div > 1);
        const int gamma = i + s * d + (d < 0 ? d : 0);
        const int first = i < j ? i : j, last = i < j ? j : i;
        const int32_t left = first == gamma ? (int32_t)(internal + gamma) : gamma;
        const int32_t right = last == gamma + 1 ? (int32_t)(internal + gamma + 1) : gamma + 1;
        nodes[i].left = left; nodes[i].right = right;
        nodes[left].parent = i; nodes[right].parent = i;
    }
    /* bounds, bottom-up: the second arrival at a node merges its children (min / max are order-free) */
    uint32_t *visit = (uint32_t *)calloc(n, sizeof(uint32_t));
    for (uint32_t k = 0; k < n; ++k) {
        int32_t node = nodes[internal + k].parent;
        while (node >= 0) {
            if (visit[node]++ == 0u) break;
            const lbvh_node *a = nodes + nodes[node].left, *b = nodes + nodes[node].right;
            for (int c = 0; c < 3; ++c) { nodes[node].lo[c] = fminf(a->lo[c], b->lo[c]); nodes[node].hi[c] = fmaxf(a->hi[c], b->hi[c]); }
            node = nodes[node].parent;
        }
    }
    free(visit);
}

static int boxes_overlap(const float *alo, const float *ahi, const float *blo, const float *bhi) {
    return !(ahi[0] < blo[0] || alo[0] > bhi[0] || ahi[1] < blo[1] || alo[1] > bhi[1] || ahi[2] < blo[2] || alo[2] > bhi[2]);
}

/* shape_kind.hpp:26-33 */
static int filter_admits(uint32_t ta, uint32_t aa, uint32_t ga_, uint32_t tb, uint32_t ab, uint32_t gb_) {
    if (((ta & ab) | (tb & aa)) == 0u) return 0;
    const int32_t ga = (int32_t)ga_, gb = (int32_t)gb_;
    return !(ga != 0 && gb != 0 && (ga > 0 ? (ga != gb && gb > 0) : ga == gb));
}
static int key_in(const uint64_t *keys, uint32_t n, uint64_t key) {
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        if (keys[mid] < key) lo = mid + 1; else if (keys[mid] > key) hi = mid; else return 1;
    }
    return 0;
}
static int cmp_u64(const void *a, const void *b) { const uint64_t x = *(const uint64_t *)a, y = *(const uint64_t *)b; return x < y ? -1 : x > y; }

/* Tree route of the candidate-pair stage: every leaf walks the tree, pairs come out unordered and are then put in
 * ascending (i << 32 | j) order.  When more pairs survive than the capacity holds, the lowest keys are kept (the
 * reference keeps whichever reserved a slot first, which its atomics do not order) and the overflow bit is set. */
void orc_find_pairs_lbvh(const orc_model *m, orc_env *e) {
    const uint32_t n = m->B;
    const uint32_t cap = m->cfg.max_pairs && m->cfg.max_pairs < m->cfg.max_contacts ? m->cfg.max_pairs : m->cfg.max_contacts;
    e->pair_count = 0;
    if (n < 2u) return;
    lbvh_node *nodes = (lbvh_node *)malloc(sizeof(lbvh_node) * (2u * n - 1u));
    uint32_t *code = (uint32_t *)malloc(sizeof(uint32_t) * n), *order = (uint32_t *)malloc(sizeof(uint32_t) * n);
    lbvh_build(n, e->aabb_lo, e->aabb_hi, nodes, code, order);
    const uint32_t internal = n - 1u;
    uint64_t *found = (uint64_t *)malloc(sizeof(uint64_t) * ((size_t)n * (n - 1u) / 2u + 1u));
    size_t nfound = 0;
    for (uint32_t k = 0; k < n; ++k) {
        const lbvh_node *mine = nodes + internal + k;
        const uint32_t a = (uint32_t)mine->left;
        int32_t stack[64];
        int top = 0;
        stack[top++] = 0;
        while (top > 0) {
            const lbvh_node *node = nodes + stack[--top];
            const int32_t children[2] = {node->left, node->right};
            for (int c = 0; c < 2; ++c) {
                const int32_t child = children[c];
                const lbvh_node *cn = nodes + child;
                if (!boxes_overlap(mine->lo, mine->hi, cn->lo, cn->hi)) continue;
                if ((uint32_t)child >= internal) {
                    const uint32_t b = (uint32_t)cn->left;
                    if (a >= b) continue;
                    if (m->body_id[a] < 0 && m->body_id[b] < 0) continue;
                    if (!filter_admits(m->contype[a], m->conaffinity[a], m->group[a], m->contype[b], m->conaffinity[b], m->group[b])) continue;
                    const uint64_t key = ((uint64_t)a << 32) | b;
                    if (m->n_excluded && key_in(m->excluded, m->n_excluded, key)) continue;
                    found[nfound++] = key;
                } else if (top < 63) stack[top++] = child;
            }
        }
    }
    qsort(found, nfound, sizeof(uint64_t), cmp_u64);
    if (nfound > cap) { e->status |= ORC_STATUS_PAIR_OVERFLOW; nfound = cap; }
    for (size_t s = 0; s < nfound; ++s) { e->pairs[2 * s] = (uint32_t)(found[s] >> 32); e->pairs[2 * s + 1] = (uint32_t)found[s]; }
    e->pair_count = (uint32_t)nfound;
    free(found); free(order); free(code); free(nodes);
}

/* Test access: the pair set of n boxes through the tree (no filters), ascending keys in out; returns the count.
 * The cases of tests/collision/test_lbvh_vs_sap_pair_set.cpp compare this with a brute-force O(n^2) pass. */
uint32_t orc_lbvh_pair_set(uint32_t n, const float *lo, const float *hi, uint64_t *out, uint32_t capacity) {
    if (n < 2u) return 0u;
    lbvh_node *nodes = (lbvh_node *)malloc(sizeof(lbvh_node) * (2u * n - 1u));
    uint32_t *code = (uint32_t *)malloc(sizeof(uint32_t) * n), *order = (uint32_t *)malloc(sizeof(uint32_t) * n);
    lbvh_build(n, lo, hi, nodes, code, order);
    const uint32_t internal = n - 1u;
    uint32_t count = 0;
    for (uint32_t k = 0; k < n; ++k) {
        const lbvh_node *mine = nodes + internal + k;
        int32_t stack[64];
        int top = 0;
        stack[top++] = 0;
        while (top > 0) {
            const lbvh_node *node = nodes + stack[--top];
            const int32_t children[2] = {node->left, node->right};
            for (int c = 0; c < 2; ++c) {
                const lbvh_node *cn = nodes + children[c];
                if (!boxes_overlap(mine->lo, mine->hi, cn->lo, cn->hi)) continue;
                if ((uint32_t)children[c] >= internal) {
                    if (mine->left < cn->left && count < capacity) out[count++] = ((uint64_t)(uint32_t)mine->left << 32) | (uint32_t)cn->left;
                } else if (top < 63) stack[top++] = children[c];
            }
        }
    }
    qsort(out, count, sizeof(uint64_t), cmp_u64);
    free(order); free(code); free(nodes);
    return count;
}
