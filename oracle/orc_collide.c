/* Oracle (test infrastructure): collidable poses, AABBs, candidate pairs, analytic manifolds.
 * Restates the reference's ops/sync_body_pose.cu, ops/broadphase.cu, ops/narrowphase_prims.cu,
 * src/collision/analytical_manifold.hpp, primitive_surface.hpp and nk/contact/contact_identity.hpp. */
#include "orc.h"
#include "orc_math.h"

/* sync_body_pose.cu:24-50 SyncLinkBodyPoseKernel */
void orc_sync_bodies(const orc_model *m, orc_env *e) {
    for (uint32_t b = 0; b < m->B; ++b) {
        const uint32_t l = m->body_to_link[b];
        if (l == ORC_NOLINK || l >= m->L) continue;
        if (m->body_geom_kind[b] != 0u) {
            float local[7];
            memcpy(local, m->body_geom_pos + 3 * b, 12); memcpy(local + 3, m->body_geom_quat + 4 * b, 16);
            pose_compose_hd(e->link_pose + 7 * l, local, e->body_pose + 7 * b);
        } else memcpy(e->body_pose + 7 * b, e->link_pose + 7 * l, 28);
    }
}

/* broadphase.cu:154-168 RotAbs */
static v3 rot_abs(quat q, v3 v) {
    v3 cx = qrot_raw(q, V3(1, 0, 0)), cy = qrot_raw(q, V3(0, 1, 0)), cz = qrot_raw(q, V3(0, 0, 1));
    return V3(fabsf(cx.x) * v.x + fabsf(cy.x) * v.y + fabsf(cz.x) * v.z,
              fabsf(cx.y) * v.x + fabsf(cy.y) * v.y + fabsf(cz.y) * v.z,
              fabsf(cx.z) * v.x + fabsf(cy.z) * v.y + fabsf(cz.z) * v.z);
}

static float query_reach(const orc_model *m) {
    /* contact_query.hpp:19-21 with zero particle thickness */
    return fmaxf(0.02f, 2.0f * (2.0f * 0.0f + m->cfg.contact_margin));
}
static float motion_radius(float base, float dt, float sa, float sb) {
    /* contact_query.hpp:27-30, relaxation kContactQueryRelaxation = 0.9 */
    return base + dt * (sa + sb) * (2.0f / 0.9f);
}

/* broadphase.cu:173-270 BuildAabbsKernel */
void orc_build_aabbs(const orc_model *m, orc_env *e) {
    const float margin = fmaxf(m->cfg.contact_margin, 0.0005f);
    const float reach = query_reach(m);
    for (uint32_t b = 0; b < m->B; ++b) {
        const float *pose = e->body_pose + 7 * b;
        const float *p = m->shape_params + 4 * b;
        v3 c = v3ld(pose), he = V3(0, 0, 0);
        quat q = qld(pose + 3);
        switch (m->shape_kind[b]) {
            case ORC_SHAPE_SPHERE: he = V3(p[0], p[0], p[0]); break;
            case ORC_SHAPE_CAPSULE: he = rot_abs(q, V3(p[0], p[0], p[0] + p[1])); break;
            case ORC_SHAPE_BOX: he = rot_abs(q, V3(p[0], p[1], p[2])); break;
            case ORC_SHAPE_CYLINDER: {      /* broadphase.cu:199-208: per world axis hh |a_i| + r sqrt(1 - a_i^2), a the cylinder's axis */
                const v3 qv = V3(q.x, q.y, q.z), ez = V3(0, 0, 1);
                const v3 tz = vscale(vcross(qv, ez), 2.0f);
                const v3 a = vadd(vadd(ez, vscale(tz, q.w)), vcross(qv, tz));
                he = V3(p[1] * fabsf(a.x) + p[0] * sqrtf(fmaxf(0.0f, 1.0f - a.x * a.x)),
                        p[1] * fabsf(a.y) + p[0] * sqrtf(fmaxf(0.0f, 1.0f - a.y * a.y)),
                        p[1] * fabsf(a.z) + p[0] * sqrtf(fmaxf(0.0f, 1.0f - a.z * a.z)));
                break;
            }
            case ORC_SHAPE_PLANE:
                v3st(e->aabb_lo + 3 * b, V3(-FLT_MAX, -FLT_MAX, -FLT_MAX));
                v3st(e->aabb_hi + 3 * b, V3(FLT_MAX, FLT_MAX, FLT_MAX));
                continue;
            default:
                v3st(e->aabb_lo + 3 * b, V3(FLT_MAX, FLT_MAX, FLT_MAX));
                v3st(e->aabb_hi + 3 * b, V3(-FLT_MAX, -FLT_MAX, -FLT_MAX));
                continue;
        }
        const float radius = sqrtf(vdot(he, he)) + 0.0f;
        const float speed = fmaxf(0.0f, vlen(v3ld(e->body_linvel + 3 * b)) + vlen(v3ld(e->body_angvel + 3 * b)) * radius);
        const float mm = fmaxf(margin, fminf(motion_radius(margin, m->cfg.dt, speed, 0.0f), reach));
        v3st(e->aabb_lo + 3 * b, V3(c.x - he.x - mm, c.y - he.y - mm, c.z - he.z - mm));
        v3st(e->aabb_hi + 3 * b, V3(c.x + he.x + mm, c.y + he.y + mm, c.z + he.z + mm));
    }
}

/* shape_kind.hpp:26-33 ShapeFilterAdmits */
static int filter_admits(uint32_t ta, uint32_t aa, uint32_t ga_, uint32_t tb, uint32_t ab, uint32_t gb_) {
    if (((ta & ab) | (tb & aa)) == 0u) return 0;
    const int32_t ga = (int32_t)ga_, gb = (int32_t)gb_;
    return !(ga != 0 && gb != 0 && (ga > 0 ? (ga != gb && gb > 0) : ga == gb));
}
static int is_excluded(const uint64_t *keys, uint32_t n, uint64_t key) {
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
        uint32_t mid = lo + ((hi - lo) >> 1);
        if (keys[mid] < key) lo = mid + 1; else if (keys[mid] > key) hi = mid; else return 1;
    }
    return 0;
}

/* broadphase.cu:276-282, 314-474, 476-678: the candidate set is every i<j whose AABBs overlap, not both
 * static, admitted by the bitmask filter and not excluded; after the canonical sort the per-env list is
 * ascending in (i<<32|j). Tree walk and all-pairs routes produce the same set. */
static void find_pairs_all(const orc_model *m, orc_env *e) {
    const uint32_t cap = m->cfg.max_pairs && m->cfg.max_pairs < m->cfg.max_contacts ? m->cfg.max_pairs : m->cfg.max_contacts;
    uint32_t count = 0;
    for (uint32_t i = 0; i < m->B; ++i) for (uint32_t j = i + 1; j < m->B; ++j) {
        const float *alo = e->aabb_lo + 3 * i, *ahi = e->aabb_hi + 3 * i, *blo = e->aabb_lo + 3 * j, *bhi = e->aabb_hi + 3 * j;
        if (ahi[0] < blo[0] || alo[0] > bhi[0] || ahi[1] < blo[1] || alo[1] > bhi[1] || ahi[2] < blo[2] || alo[2] > bhi[2]) continue;
        if (m->body_id[i] < 0 && m->body_id[j] < 0) continue;
        if (!filter_admits(m->contype[i], m->conaffinity[i], m->group[i], m->contype[j], m->conaffinity[j], m->group[j])) continue;
        if (m->n_excluded && is_excluded(m->excluded, m->n_excluded, ((uint64_t)i << 32) | j)) continue;
        if (count < cap) { e->pairs[2 * count] = i; e->pairs[2 * count + 1] = j; ++count; }
        else e->status |= ORC_STATUS_PAIR_OVERFLOW;
    }
    e->pair_count = count;
}

/* broadphase.cu:581, 608: the all-pairs kernel replaces tree build + walk while B^2 E <= 2^20 (kAllPairsItems); the
 * world can also pin either route, for the tests that show the two agree. */
void orc_find_pairs(const orc_model *m, orc_env *e) {
    const uint64_t items = (uint64_t)m->B * m->B * (m->env_count ? m->env_count : 1u);
    const int tree = m->broadphase == 2u || (m->broadphase == 0u && items > (1u << 20));
    if (tree) orc_find_pairs_lbvh(m, e); else find_pairs_all(m, e);
}

/* ---- analytic manifolds ---- */
typedef struct { v3 cx, cy, cz, t; } frame;
typedef struct { v3 he; float radius, hh; frame f; } prim;
typedef struct { v3 pos, n; float pen; uint64_t key; } cpt;
typedef struct { uint32_t count; cpt p[4]; } manifold;
typedef struct { v3 pos; float pen; uint32_t feat; } cand;

static v3 f_l2w(const frame *f, v3 l) {
    return V3(f->cx.x * l.x + f->cy.x * l.y + f->cz.x * l.z + f->t.x,
              f->cx.y * l.x + f->cy.y * l.y + f->cz.y * l.z + f->t.y,
              f->cx.z * l.x + f->cy.z * l.y + f->cz.z * l.z + f->t.z);
}
static v3 f_w2l(const frame *f, v3 w) {
    v3 d = vsub(w, f->t);
    return V3(vdot(d, f->cx), vdot(d, f->cy), vdot(d, f->cz));
}
static v3 f_dir(const frame *f, v3 l) {
    return V3(f->cx.x * l.x + f->cy.x * l.y + f->cz.x * l.z, f->cx.y * l.x + f->cy.y * l.y + f->cz.y * l.z,
              f->cx.z * l.x + f->cy.z * l.y + f->cz.z * l.z);
}
static v3 f_axis(const frame *f, int k) { return k == 0 ? f->cx : (k == 1 ? f->cy : f->cz); }
static v3 norm_or(v3 v, v3 fb) { float l = vlen(v); if (l < 1.0e-12f) return fb; return V3(v.x / l, v.y / l, v.z / l); }
static void add_pt(manifold *o, v3 pos, v3 n, float pen, uint64_t key) {
    if (o->count < 4u) { cpt c = {pos, n, pen, key}; o->p[o->count++] = c; }
}

/* analytical_manifold.hpp:273-311 ReduceAndEmit */
static void reduce_emit(cand *c, int n, v3 normal, manifold *o) {
    if (n <= 0) return;
    const int keep = n < 4 ? n : 4;
    for (int s = 0; s < keep; ++s) {
        int best = s;
        for (int i = s + 1; i < n; ++i)
            if (c[i].pen > c[best].pen || (c[i].pen == c[best].pen && c[i].feat < c[best].feat)) best = i;
        cand t = c[s]; c[s] = c[best]; c[best] = t;
    }
    for (int i = 1; i < keep; ++i) {
        cand key = c[i]; int j = i - 1;
        while (j >= 0 && c[j].feat > key.feat) { c[j + 1] = c[j]; --j; }
        c[j + 1] = key;
    }
    o->count = 0;
    for (int i = 0; i < keep; ++i) add_pt(o, c[i].pos, normal, c[i].pen, c[i].feat);
}

/* analytical_manifold.hpp:337-401 ReduceAndEmitSpread */
static void reduce_emit_spread(cand *c, int n, v3 normal, manifold *o) {
    o->count = 0;
    if (n <= 0) return;
    if (n <= 4) {
        for (int i = 1; i < n; ++i) {
            cand key = c[i]; int j = i - 1;
            while (j >= 0 && c[j].feat > key.feat) { c[j + 1] = c[j]; --j; }
            c[j + 1] = key;
        }
        for (int i = 0; i < n; ++i) add_pt(o, c[i].pos, normal, c[i].pen, c[i].feat);
        return;
    }
    int kept[4]; int used[24] = {0};
    int seed = 0;
    for (int i = 1; i < n; ++i) if (c[i].pen > c[seed].pen) seed = i;
    kept[0] = seed; used[seed] = 1;
    int nk = 1;
    for (int s = 1; s < 4; ++s) {
        int best = -1; float best_mind = -1.0f;
        for (int i = 0; i < n; ++i) {
            if (used[i]) continue;
            float mind = 3.4e38f;
            for (int t = 0; t < s; ++t) { v3 d = vsub(c[i].pos, c[kept[t]].pos); float dd = vdot(d, d); if (dd < mind) mind = dd; }
            if (mind > best_mind) { best_mind = mind; best = i; }
        }
        if (best < 0) break;
        kept[s] = best; used[best] = 1; nk = s + 1;
    }
    for (int i = 1; i < 4; ++i) {
        int key = kept[i], j = i - 1;
        while (j >= 0 && c[kept[j]].feat > c[key].feat) { kept[j + 1] = kept[j]; --j; }
        kept[j + 1] = key;
    }
    (void)nk;
    for (int i = 0; i < 4; ++i) add_pt(o, c[kept[i]].pos, normal, c[kept[i]].pen, c[kept[i]].feat);
}

/* analytical_manifold.hpp:416-428 */
static void sphere_sphere(const prim *a, const prim *b, manifold *o, float query) {
    v3 delta = vsub(a->f.t, b->f.t);
    float dist = vlen(delta), pen = (a->radius + b->radius) - dist;
    if (pen <= -query) return;
    v3 n = norm_or(delta, V3(0, 1, 0));
    add_pt(o, vadd(b->f.t, vscale(n, b->radius - 0.5f * pen)), n, pen, 0);
}

/* primitive_surface.hpp:28-88 box and capsule branches */
static int surface_box(v3 he, v3 p, float *dist, v3 *normal, v3 *point) {
    if (!(he.x >= 0.0f && he.y >= 0.0f && he.z >= 0.0f)) return 0;
    v3 cl = V3(fmaxf(-he.x, fminf(p.x, he.x)), fmaxf(-he.y, fminf(p.y, he.y)), fmaxf(-he.z, fminf(p.z, he.z)));
    v3 off = vsub(p, cl);
    float len = sqrtf(vdot(off, off));
    if (len > 0.0f) { *dist = len; *normal = V3(off.x / len, off.y / len, off.z / len); }
    else {
        v3 d = V3(fabsf(p.x) - he.x, fabsf(p.y) - he.y, fabsf(p.z) - he.z);
        if (d.x >= d.y && d.x >= d.z) { *dist = d.x; *normal = V3(p.x < 0.0f ? -1.0f : 1.0f, 0, 0); }
        else if (d.y >= d.z) { *dist = d.y; *normal = V3(0, p.y < 0.0f ? -1.0f : 1.0f, 0); }
        else { *dist = d.z; *normal = V3(0, 0, p.z < 0.0f ? -1.0f : 1.0f); }
    }
    *point = vsub(p, vscale(*normal, *dist));
    return 1;
}
static int surface_capsule(float r, float hh, v3 p, float *dist, v3 *normal, v3 *point) {
    if (!(r >= 0.0f) || !(hh >= 0.0f)) return 0;
    v3 off = p;
    off.z -= fmaxf(-hh, fminf(p.z, hh));
    float len = sqrtf(vdot(off, off));
    *normal = V3(1, 0, 0);
    if (len > 0.0f) *normal = V3(off.x / len, off.y / len, off.z / len);
    *dist = len - r;
    *point = vsub(p, vscale(*normal, *dist));
    return 1;
}

/* analytical_manifold.hpp:434-448 */
static void sphere_box(const prim *s, const prim *box, manifold *o, float query) {
    float dist; v3 n, pt;
    if (!surface_box(box->he, f_w2l(&box->f, s->f.t), &dist, &n, &pt)) return;
    float pen = s->radius - dist;
    if (pen <= -query) return;
    v3 nw = f_dir(&box->f, n);
    add_pt(o, vsub(f_l2w(&box->f, pt), vscale(nw, 0.5f * pen)), nw, pen, 0);
}
/* analytical_manifold.hpp:451-462 */
static void sphere_plane(const prim *s, const prim *pl, manifold *o, float query) {
    v3 n = norm_or(pl->f.cz, V3(0, 0, 1));
    float sd = vdot(vsub(s->f.t, pl->f.t), n), pen = s->radius - sd;
    if (pen <= -query) return;
    add_pt(o, vsub(s->f.t, vscale(n, s->radius - 0.5f * pen)), n, pen, 0);
}
/* analytical_manifold.hpp:469-492 */
static void box_plane(const prim *box, const prim *pl, manifold *o, float query) {
    v3 n = norm_or(pl->f.cz, V3(0, 0, 1));
    cand c[8]; int nc = 0;
    for (uint32_t k = 0; k < 8u; ++k) {
        float sx = (k & 1u) ? 1.0f : -1.0f, sy = (k & 2u) ? 1.0f : -1.0f, sz = (k & 4u) ? 1.0f : -1.0f;
        v3 cw = f_l2w(&box->f, V3(sx * box->he.x, sy * box->he.y, sz * box->he.z));
        float sd = vdot(vsub(cw, pl->f.t), n);
        if (sd < query) { c[nc].pos = vsub(cw, vscale(n, 0.5f * sd)); c[nc].pen = -sd; c[nc].feat = k; ++nc; }
    }
    reduce_emit(c, nc, n, o);
}
/* analytical_manifold.hpp:738-758 */
static void capsule_plane(const prim *cap, const prim *pl, manifold *o, float query) {
    v3 n = norm_or(pl->f.cz, V3(0, 0, 1));
    v3 ends[2] = {vadd(cap->f.t, vscale(cap->f.cz, cap->hh)), vsub(cap->f.t, vscale(cap->f.cz, cap->hh))};
    cand c[2]; int nc = 0;
    for (uint32_t k = 0; k < 2u; ++k) {
        float sd = vdot(vsub(ends[k], pl->f.t), n) - cap->radius;
        if (sd < query) { c[nc].pos = vsub(ends[k], vscale(n, cap->radius + 0.5f * sd)); c[nc].pen = -sd; c[nc].feat = k; ++nc; }
    }
    reduce_emit(c, nc, n, o);
}
/* analytical_manifold.hpp:764-778 */
static void capsule_sphere(const prim *cap, const prim *s, manifold *o, float query) {
    float dist; v3 n, pt;
    if (!surface_capsule(cap->radius, cap->hh, f_w2l(&cap->f, s->f.t), &dist, &n, &pt)) return;
    float pen = s->radius - dist;
    if (pen <= -query) return;
    v3 nw = vscale(f_dir(&cap->f, n), -1.0f);
    add_pt(o, vadd(f_l2w(&cap->f, pt), vscale(nw, 0.5f * pen)), nw, pen, 0);
}
/* primitive_surface.hpp:89-114 cylinder branch: features 0 bottom cap, 1 side, 2 top cap, 3 bottom rim, 4 top rim */
static int surface_cylinder(float r, float hh, v3 p, float *dist, v3 *normal, v3 *point, uint32_t *feature) {
    if (!(r >= 0.0f && hh >= 0.0f)) return 0;
    const float rho = sqrtf(p.x * p.x + p.y * p.y);
    const v3 radial = rho > 0.0f ? V3(p.x / rho, p.y / rho, 0.0f) : V3(1.0f, 0.0f, 0.0f);
    const v3 axial = V3(0.0f, 0.0f, p.z < 0.0f ? -1.0f : 1.0f);
    const float side = rho - r, cap = fabsf(p.z) - hh;
    if (side > 0.0f && cap > 0.0f) {
        *dist = sqrtf(side * side + cap * cap);
        const v3 sum = vadd(vscale(radial, side), vscale(axial, cap));
        *normal = V3(sum.x / *dist, sum.y / *dist, sum.z / *dist);
        *feature = p.z < 0.0f ? 3u : 4u;
    } else if (side > cap) { *dist = side; *normal = radial; *feature = 1u; }
    else { *dist = cap; *normal = axial; *feature = p.z < 0.0f ? 0u : 2u; }
    *point = vsub(p, vscale(*normal, *dist));
    return 1;
}
/* analytical_manifold.hpp:780-816: the lower cap's octagon and deepest point when a cap faces the plane, else each cap's
 * deepest rim point */
static void cylinder_plane(const prim *cyl, const prim *pl, manifold *o, float query) {
    static const float kc[8] = {1.0f, 0.70710678f, 0.0f, -0.70710678f, -1.0f, -0.70710678f, 0.0f, 0.70710678f};
    static const float ks[8] = {0.0f, 0.70710678f, 1.0f, 0.70710678f, 0.0f, -0.70710678f, -1.0f, -0.70710678f};
    const v3 n = norm_or(pl->f.cz, V3(0, 0, 1));
    const v3 axis = cyl->f.cz;
    const float d = vdot(axis, n);
    const int on_cap = (d < 0.0f ? -d : d) >= 0.95f;
    const v3 down = norm_or(vsub(vscale(axis, d), n), cyl->f.cx);
    cand c[10]; int nc = 0;
    for (int cap = 0; cap < 2; ++cap) {
        if (on_cap && (cap == 0) == (d > 0.0f)) continue;
        const v3 center = vadd(cyl->f.t, vscale(axis, cap == 0 ? cyl->hh : -cyl->hh));
        for (int k = -1; k < (on_cap ? 8 : 0); ++k) {
            const v3 dir = k < 0 ? down : vadd(vscale(cyl->f.cx, kc[k]), vscale(cyl->f.cy, ks[k]));
            const v3 p = vadd(center, vscale(dir, cyl->radius));
            const float sd = vdot(vsub(p, pl->f.t), n);
            if (sd >= query) continue;
            c[nc].pos = vsub(p, vscale(n, sd * 0.5f)); c[nc].pen = -sd; c[nc].feat = (uint32_t)(k < 0 ? cap : 2 + cap * 8 + k); ++nc;
        }
    }
    reduce_emit_spread(c, nc, n, o);
}
/* analytical_manifold.hpp:818-834 */
static void cylinder_sphere(const prim *cyl, const prim *s, manifold *o, float query) {
    float dist; v3 n, pt; uint32_t feature;
    if (!surface_cylinder(cyl->radius, cyl->hh, f_w2l(&cyl->f, s->f.t), &dist, &n, &pt, &feature)) return;
    float pen = s->radius - dist;
    if (pen <= -query) return;
    v3 nw = vscale(f_dir(&cyl->f, n), -1.0f);
    add_pt(o, vadd(f_l2w(&cyl->f, pt), vscale(nw, 0.5f * pen)), nw, pen, feature);
}
/* analytical_manifold.hpp:841-896 */
static float closest_seg_seg(v3 p1, v3 q1, v3 p2, v3 q2, v3 *c1, v3 *c2) {
    v3 d1 = vsub(q1, p1), d2 = vsub(q2, p2), r = vsub(p1, p2);
    float a = vdot(d1, d1), e = vdot(d2, d2), f = vdot(d2, r), s = 0.0f, t = 0.0f;
    const float eps = 1.0e-12f;
    if (a <= eps && e <= eps) { s = t = 0.0f; }
    else if (a <= eps) { s = 0.0f; t = f / e; t = t < 0.0f ? 0.0f : (t > 1.0f ? 1.0f : t); }
    else {
        float c = vdot(d1, r);
        if (e <= eps) { t = 0.0f; s = -c / a; s = s < 0.0f ? 0.0f : (s > 1.0f ? 1.0f : s); }
        else {
            float b = vdot(d1, d2), denom = a * e - b * b;
            if (denom > eps) { s = (b * f - c * e) / denom; s = s < 0.0f ? 0.0f : (s > 1.0f ? 1.0f : s); }
            else s = 0.0f;
            t = (b * s + f) / e;
            if (t < 0.0f) { t = 0.0f; s = -c / a; s = s < 0.0f ? 0.0f : (s > 1.0f ? 1.0f : s); }
            else if (t > 1.0f) { t = 1.0f; s = (b - c) / a; s = s < 0.0f ? 0.0f : (s > 1.0f ? 1.0f : s); }
        }
    }
    *c1 = vadd(p1, vscale(d1, s)); *c2 = vadd(p2, vscale(d2, t));
    v3 dv = vsub(*c1, *c2);
    return vdot(dv, dv);
}
/* analytical_manifold.hpp:905-932 */
static void capsule_capsule(const prim *a, const prim *b, manifold *o, float query) {
    v3 axa = a->f.cz, axb = b->f.cz, ca, cb;
    float d2 = closest_seg_seg(vadd(a->f.t, vscale(axa, a->hh)), vsub(a->f.t, vscale(axa, a->hh)),
                               vadd(b->f.t, vscale(axb, b->hh)), vsub(b->f.t, vscale(axb, b->hh)), &ca, &cb);
    float dist = sqrtf(d2), pen = (a->radius + b->radius) - dist;
    if (pen <= -query) return;
    v3 n = norm_or(vsub(ca, cb), norm_or(vcross(axa, axb), V3(0, 1, 0)));
    v3 sa = vsub(ca, vscale(n, a->radius)), sb = vadd(cb, vscale(n, b->radius));
    add_pt(o, vscale(vadd(sa, sb), 0.5f), n, pen, 0);
}

typedef struct { v3 v[8]; uint32_t feat[8]; int count; } clip_poly;
static void poly_add(clip_poly *p, v3 v, uint32_t f) { if (p->count < 8) { p->v[p->count] = v; p->feat[p->count] = f; ++p->count; } }
/* analytical_manifold.hpp:224-250 */
static clip_poly clip_plane(const clip_poly *in, v3 pp, v3 pn) {
    clip_poly out; out.count = 0;
    for (int i = 0; i < in->count; ++i) {
        int j = (i + 1) % in->count;
        v3 cur = in->v[i], nxt = in->v[j];
        float dc = vdot(vsub(cur, pp), pn), dn = vdot(vsub(nxt, pp), pn);
        int ci = dc <= 0.0f, ni = dn <= 0.0f;
        if (ci) poly_add(&out, cur, in->feat[i]);
        if (ci != ni) {
            float t = dc / (dc - dn);
            poly_add(&out, V3(cur.x + (nxt.x - cur.x) * t, cur.y + (nxt.y - cur.y) * t, cur.z + (nxt.z - cur.z) * t), in->feat[i]);
        }
    }
    return out;
}
static float fabs_dot(v3 a, v3 b) { float d = vdot(a, b); return d < 0.0f ? -d : d; }

/* analytical_manifold.hpp:503-734 */
static void box_box(const prim *A, const prim *B, manifold *o, float query) {
    v3 ha = A->he, hb = B->he, dpos = vsub(B->f.t, A->f.t);
    v3 ax[3] = {A->f.cx, A->f.cy, A->f.cz}, bx[3] = {B->f.cx, B->f.cy, B->f.cz};
    float R[3][3], AbsR[3][3];
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) { R[i][j] = vdot(ax[i], bx[j]); AbsR[i][j] = (R[i][j] < 0.0f ? -R[i][j] : R[i][j]) + 1.0e-6f; }
    const float ea[3] = {ha.x, ha.y, ha.z}, eb[3] = {hb.x, hb.y, hb.z};
    const float dA[3] = {vdot(dpos, ax[0]), vdot(dpos, ax[1]), vdot(dpos, ax[2])};
    float min_pen = 3.4e38f; int best_axis = -1; v3 best_n = V3(0, 1, 0);
    const float bias = 1.0e-5f;
    for (int i = 0; i < 3; ++i) {
        float ra = ea[i], rb = eb[0] * AbsR[i][0] + eb[1] * AbsR[i][1] + eb[2] * AbsR[i][2];
        float s = dA[i] < 0.0f ? -dA[i] : dA[i], pen = (ra + rb) - s;
        if (pen <= -query) return;
        if (pen < min_pen - bias) { min_pen = pen; best_axis = i; best_n = dA[i] < 0.0f ? vneg(ax[i]) : ax[i]; }
    }
    for (int j = 0; j < 3; ++j) {
        float ra = ea[0] * AbsR[0][j] + ea[1] * AbsR[1][j] + ea[2] * AbsR[2][j], rb = eb[j];
        float dB = vdot(dpos, bx[j]), s = dB < 0.0f ? -dB : dB, pen = (ra + rb) - s;
        if (pen <= -query) return;
        if (pen < min_pen - bias) { min_pen = pen; best_axis = 3 + j; best_n = dB < 0.0f ? vneg(bx[j]) : bx[j]; }
    }
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) {
        v3 Lx = vcross(ax[i], bx[j]);
        float ll = vlen(Lx);
        if (ll < 1.0e-6f) continue;
        Lx = V3(Lx.x / ll, Lx.y / ll, Lx.z / ll);
        float ra = ea[0] * fabs_dot(ax[0], Lx) + ea[1] * fabs_dot(ax[1], Lx) + ea[2] * fabs_dot(ax[2], Lx);
        float rb = eb[0] * fabs_dot(bx[0], Lx) + eb[1] * fabs_dot(bx[1], Lx) + eb[2] * fabs_dot(bx[2], Lx);
        float s = vdot(dpos, Lx), sa = s < 0.0f ? -s : s, pen = (ra + rb) - sa;
        if (pen <= -query) return;
        if (pen < min_pen - bias) { min_pen = pen; best_axis = 6 + i * 3 + j; best_n = s < 0.0f ? vneg(Lx) : Lx; }
    }
    if (best_axis < 0) return;
    if (best_axis >= 6) {
        int i = (best_axis - 6) / 3, j = (best_axis - 6) % 3;
        v3 pa = A->f.t, pb = B->f.t;
        for (int k = 0; k < 3; ++k) { if (k == i) continue; float sg = vdot(ax[k], best_n) >= 0.0f ? 1.0f : -1.0f; pa = vadd(pa, vscale(ax[k], sg * ea[k])); }
        for (int k = 0; k < 3; ++k) { if (k == j) continue; float sg = vdot(bx[k], best_n) >= 0.0f ? -1.0f : 1.0f; pb = vadd(pb, vscale(bx[k], sg * eb[k])); }
        v3 ed = ax[i], fd = bx[j], r = vsub(pa, pb);
        float aa = 1.0f, bb = vdot(ed, fd), cc = 1.0f, dd = vdot(ed, r), ee = vdot(fd, r), denom = aa * cc - bb * bb;
        float sN = 0.0f, tN = 0.0f;
        if (denom > 1.0e-9f) { sN = (bb * ee - cc * dd) / denom; tN = (aa * ee - bb * dd) / denom; }
        float sC = sN < -ea[i] ? -ea[i] : (sN > ea[i] ? ea[i] : sN), tC = tN < -eb[j] ? -eb[j] : (tN > eb[j] ? eb[j] : tN);
        v3 ca = vadd(pa, vscale(ed, sC)), cb = vadd(pb, vscale(fd, tC));
        add_pt(o, vscale(vadd(ca, cb), 0.5f), best_n, min_pen, 0xE0000000ull | ((uint64_t)i << 4) | (uint64_t)j);
        return;
    }
    const int ref_is_A = best_axis < 3, ref_axis = ref_is_A ? best_axis : best_axis - 3;
    const frame *Rf = ref_is_A ? &A->f : &B->f, *If = ref_is_A ? &B->f : &A->f;
    v3 rhe = ref_is_A ? ha : hb, ihe = ref_is_A ? hb : ha;
    v3 refN = f_axis(Rf, ref_axis);
    if (vdot(vsub(If->t, Rf->t), refN) < 0.0f) refN = vneg(refN);
    int inc_axis = 0; float best_dot = 3.4e38f, inc_sign = 1.0f;
    for (int k = 0; k < 3; ++k) {
        float d = vdot(f_axis(If, k), refN), ad = d < 0.0f ? -d : d;
        if (-ad < best_dot) { best_dot = -ad; inc_axis = k; inc_sign = d < 0.0f ? 1.0f : -1.0f; }
    }
    int iu = (inc_axis + 1) % 3, iv = (inc_axis + 2) % 3;
    v3 ifc = vadd(If->t, vscale(f_axis(If, inc_axis), inc_sign * vcomp(ihe, inc_axis)));
    v3 iuw = f_axis(If, iu), ivw = f_axis(If, iv);
    float iue = vcomp(ihe, iu), ive = vcomp(ihe, iv);
    clip_poly poly; poly.count = 0;
    const float su[4] = {-1, 1, 1, -1}, sv[4] = {-1, -1, 1, 1};
    for (uint32_t k = 0; k < 4u; ++k)
        poly_add(&poly, vadd(vadd(ifc, vscale(iuw, su[k] * iue)), vscale(ivw, sv[k] * ive)), ((uint32_t)inc_axis << 4) | k);
    int ru = (ref_axis + 1) % 3, rv = (ref_axis + 2) % 3;
    v3 ruw = f_axis(Rf, ru), rvw = f_axis(Rf, rv);
    float rue = vcomp(rhe, ru), rve = vcomp(rhe, rv);
    v3 rfc = vadd(Rf->t, vscale(refN, vcomp(rhe, ref_axis)));
    poly = clip_plane(&poly, vadd(rfc, vscale(ruw, rue)), ruw);
    poly = clip_plane(&poly, vsub(rfc, vscale(ruw, rue)), vneg(ruw));
    poly = clip_plane(&poly, vadd(rfc, vscale(rvw, rve)), rvw);
    poly = clip_plane(&poly, vsub(rfc, vscale(rvw, rve)), vneg(rvw));
    cand c[8]; int nc = 0;
    for (int k = 0; k < poly.count; ++k) {
        float depth = vdot(vsub(rfc, poly.v[k]), refN);
        if (depth >= -query) {
            v3 onref = vadd(poly.v[k], vscale(refN, depth));
            c[nc].pos = vscale(vadd(poly.v[k], onref), 0.5f); c[nc].pen = depth; c[nc].feat = (uint32_t)k; ++nc;
        }
    }
    v3 nA = ref_is_A ? vneg(refN) : refN;
    if (nc == 0) { add_pt(o, vadd(ifc, vscale(refN, min_pen * 0.5f)), nA, min_pen, (uint64_t)inc_axis << 4); return; }
    reduce_emit_spread(c, nc, nA, o);
}

/* analytical_manifold.hpp:934-966 PrimitivePair */
static int primitive_pair(uint32_t ka, const prim *a, uint32_t kb, const prim *b, float query, manifold *o) {
    o->count = 0;
    if (ka == ORC_SHAPE_SPHERE && kb == ORC_SHAPE_SPHERE) { sphere_sphere(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_SPHERE && kb == ORC_SHAPE_BOX) { sphere_box(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_SPHERE && kb == ORC_SHAPE_PLANE) { sphere_plane(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_BOX && kb == ORC_SHAPE_PLANE) { box_plane(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_BOX && kb == ORC_SHAPE_BOX) { box_box(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_CAPSULE && kb == ORC_SHAPE_PLANE) { capsule_plane(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_CAPSULE && kb == ORC_SHAPE_SPHERE) { capsule_sphere(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_CAPSULE && kb == ORC_SHAPE_CAPSULE) { capsule_capsule(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_CYLINDER && kb == ORC_SHAPE_PLANE) { cylinder_plane(a, b, o, query); return 1; }
    if (ka == ORC_SHAPE_CYLINDER && kb == ORC_SHAPE_SPHERE) { cylinder_sphere(a, b, o, query); return 1; }
    int done = 1;
    if (ka == ORC_SHAPE_BOX && kb == ORC_SHAPE_SPHERE) sphere_box(b, a, o, query);
    else if (ka == ORC_SHAPE_PLANE && kb == ORC_SHAPE_SPHERE) sphere_plane(b, a, o, query);
    else if (ka == ORC_SHAPE_PLANE && kb == ORC_SHAPE_BOX) box_plane(b, a, o, query);
    else if (ka == ORC_SHAPE_PLANE && kb == ORC_SHAPE_CAPSULE) capsule_plane(b, a, o, query);
    else if (ka == ORC_SHAPE_SPHERE && kb == ORC_SHAPE_CAPSULE) capsule_sphere(b, a, o, query);
    else if (ka == ORC_SHAPE_PLANE && kb == ORC_SHAPE_CYLINDER) cylinder_plane(b, a, o, query);
    else if (ka == ORC_SHAPE_SPHERE && kb == ORC_SHAPE_CYLINDER) cylinder_sphere(b, a, o, query);
    else done = 0;
    if (done) for (uint32_t i = 0; i < o->count; ++i) o->p[i].n = vneg(o->p[i].n);
    return done;
}

/* contact_identity.hpp:118-160 */
static uint64_t hash_word(uint64_t h, uint64_t w) { h ^= w; h *= 1099511628211ull; return h; }
static int32_t quantize(float v) { float s = v * 4096.0f; float r = s >= 0.0f ? s + 0.5f : s - 0.5f; return (int32_t)r; }
static uint64_t feature_token(uint32_t feature, v3 p) {
    if (feature != 0xffffffffu) return 0x8000000000000000ull | (uint64_t)feature;
    uint64_t h = 1469598103934665603ull;
    h = hash_word(h, (uint32_t)quantize(p.x)); h = hash_word(h, (uint32_t)quantize(p.y)); h = hash_word(h, (uint32_t)quantize(p.z));
    return h & 0x7fffffffffffffffull;
}
static v3 inv_xf_point(const float *pose, v3 w) {
    /* prims_types.cuh:103-111 */
    v3 v = vsub(w, v3ld(pose));
    quat q = qld(pose + 3);
    v3 qv = V3(-q.x, -q.y, -q.z);
    v3 t = vscale(vcross(qv, v), 2.0f);
    return vadd(vadd(v, vscale(t, q.w)), vcross(qv, t));
}

static prim make_prim(const orc_model *m, const orc_env *e, uint32_t b) {
    /* narrowphase_prims.cu:34-46 MakePrim */
    prim p;
    quat q = qld(e->body_pose + 7 * b + 3);
    p.f.cx = qrot_raw(q, V3(1, 0, 0)); p.f.cy = qrot_raw(q, V3(0, 1, 0)); p.f.cz = qrot_raw(q, V3(0, 0, 1));
    p.f.t = v3ld(e->body_pose + 7 * b);
    const float *s = m->shape_params + 4 * b;
    p.radius = s[0]; p.hh = s[1]; p.he = V3(s[0], s[1], s[2]);
    return p;
}
static float body_speed(const orc_env *e, uint32_t b) {
    /* narrowphase_prims.cu:234-243 */
    v3 c = v3ld(e->body_pose + 7 * b);
    v3 lo = vsub(v3ld(e->aabb_lo + 3 * b), c), hi = vsub(v3ld(e->aabb_hi + 3 * b), c);
    v3 ext = V3(fmaxf(fabsf(lo.x), fabsf(hi.x)), fmaxf(fabsf(lo.y), fabsf(hi.y)), fmaxf(fabsf(lo.z), fabsf(hi.z)));
    v3 w = v3ld(e->body_angvel + 3 * b);
    return fmaxf(0.0f, vlen(v3ld(e->body_linvel + 3 * b)) + sqrtf(vdot(w, w) * vdot(ext, ext)));
}

/* narrowphase_prims.cu:181-366 PairDrivenNarrowphaseKernel<false>, speculative law */
void orc_narrowphase(const orc_model *m, orc_env *e) {
    const float separation = fmaxf(m->cfg.contact_margin, 0.0005f);
    const float reach = query_reach(m);
    e->contact_points = 0;
    for (uint32_t s = 0; s < m->cfg.max_contacts; ++s) {
        e->ccount[s] = 0;
        if (s >= e->pair_count) continue;
        const uint32_t a = e->pairs[2 * s], b = e->pairs[2 * s + 1];
        const prim pa = make_prim(m, e, a), pb = make_prim(m, e, b);
        const float query = fmaxf(separation, fminf(motion_radius(2.0f * separation, m->cfg.dt, body_speed(e, a), body_speed(e, b)), reach));
        manifold mf;
        primitive_pair(m->shape_kind[a], &pa, m->shape_kind[b], &pb, query, &mf);
        e->ccount[s] = mf.count;
        for (uint32_t i = 0; i < mf.count; ++i) {
            const uint32_t at = s * 4u + i;
            v3st(e->cpoint + 3 * at, mf.p[i].pos);
            v3st(e->cnormal + 3 * at, mf.p[i].n);
            e->cdepth[at] = mf.p[i].pen + separation;
            /* contact identity: sides are already ordered (a < b) */
            v3 la = inv_xf_point(e->body_pose + 7 * a, mf.p[i].pos), lb = inv_xf_point(e->body_pose + 7 * b, mf.p[i].pos);
            const uint32_t feature = mf.p[i].key == 0u ? 0xffffffffu : (uint32_t)mf.p[i].key;
            uint64_t h = 1469598103934665603ull;
            h = hash_word(h, feature_token(feature, la));
            h = hash_word(h, feature_token(feature, lb));
            h = hash_word(h, i);
            h = hash_word(h, 0u);
            h = hash_word(h, 0u);
            e->cid_pair[at] = ((uint64_t)(a & 0x0fffffffu) << 32) | (uint64_t)(b & 0x0fffffffu);
            e->cid_feature[at] = h;
        }
        e->contact_points += mf.count;
    }
}

/* Known-answer access for tests: the contact identity of one point (nk/contact/contact_identity.hpp), as the
 * narrowphase composes it: feature 0xffffffff means "no stable feature", then the quantised local points decide. */
uint64_t orc_contact_identity(uint32_t feature, const float *local_a, const float *local_b, uint32_t slot) {
    uint64_t h = 1469598103934665603ull;
    h = hash_word(h, feature_token(feature, v3ld(local_a)));
    h = hash_word(h, feature_token(feature, v3ld(local_b)));
    h = hash_word(h, slot);
    h = hash_word(h, 0u);
    h = hash_word(h, 0u);
    return h;
}

/* Known-answer access for tests: one analytic pair. pose = xyz + wxyz, params = shape_params (4).
 * out: count, then per point position(3) normal(3) penetration(1) (raw manifold, no separation shell). */
int orc_manifold(uint32_t kind_a, const float *pose_a, const float *params_a, uint32_t kind_b, const float *pose_b,
                 const float *params_b, float query, float *out) {
    prim p[2];
    const float *poses[2] = {pose_a, pose_b}, *pars[2] = {params_a, params_b};
    for (int k = 0; k < 2; ++k) {
        quat q = qld(poses[k] + 3);
        p[k].f.cx = qrot_raw(q, V3(1, 0, 0)); p[k].f.cy = qrot_raw(q, V3(0, 1, 0)); p[k].f.cz = qrot_raw(q, V3(0, 0, 1));
        p[k].f.t = v3ld(poses[k]);
        p[k].radius = pars[k][0]; p[k].hh = pars[k][1]; p[k].he = V3(pars[k][0], pars[k][1], pars[k][2]);
    }
    manifold mf;
    primitive_pair(kind_a, &p[0], kind_b, &p[1], query, &mf);
    for (uint32_t i = 0; i < mf.count; ++i) {
        v3st(out + 7 * i, mf.p[i].pos); v3st(out + 7 * i + 3, mf.p[i].n); out[7 * i + 6] = mf.p[i].pen;
    }
    return (int)mf.count;
}

/* Differential-test access: one analytic pair given world frames (cx, cy, cz, t: 12 floats) instead of poses, so that
 * this restatement and the reference's own header evaluate the same inputs bit for bit.  out as orc_manifold;
 * keys: the stable feature key of each point.  Returns the point count, -1 for a pair kind without a handler. */
int orc_manifold_frames(uint32_t kind_a, const float *frame_a, const float *params_a, uint32_t kind_b, const float *frame_b,
                        const float *params_b, float query, float *out, uint64_t *keys) {
    prim p[2];
    const float *frames[2] = {frame_a, frame_b}, *pars[2] = {params_a, params_b};
    for (int k = 0; k < 2; ++k) {
        p[k].f.cx = v3ld(frames[k]); p[k].f.cy = v3ld(frames[k] + 3); p[k].f.cz = v3ld(frames[k] + 6); p[k].f.t = v3ld(frames[k] + 9);
        p[k].radius = pars[k][0]; p[k].hh = pars[k][1]; p[k].he = V3(pars[k][0], pars[k][1], pars[k][2]);
    }
    manifold mf;
    if (!primitive_pair(kind_a, &p[0], kind_b, &p[1], query, &mf)) return -1;
    for (uint32_t i = 0; i < mf.count; ++i) {
        v3st(out + 7 * i, mf.p[i].pos); v3st(out + 7 * i + 3, mf.p[i].n); out[7 * i + 6] = mf.p[i].pen;
        keys[i] = mf.p[i].key;
    }
    return (int)mf.count;
}
