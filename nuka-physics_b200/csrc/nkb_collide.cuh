// Warp-per-env collision stages: collidable poses, free-body velocity kick, inflated AABBs, candidate pairs and
// analytic contact manifolds.  Quantities follow the reference's ops/sync_body_pose.cu:24-50,
// ops/articulation.cu:1019-1051, ops/broadphase.cu:173-270 and :276-474 (pair predicate),
// ops/narrowphase_prims.cu:181-366 and src/collision/analytical_manifold.hpp:416-966.
#pragma once
#include "nkb_dynamics.cuh"

namespace nkb {

NKB_DEV float* sm_bpose(const Env& e, uint32_t b) { return e.sm + e.lay->bpose + 7u * b; }

NKB_DEV uint32_t free_slot(const Env& e, uint32_t b) { return __ldg(e.t->free_slot + b); }
// velocities live in the free-body slots; every link-mirror or static row shares the last slot, which holds zeros
NKB_DEV float* sm_bvel(const Env& e, uint32_t b) { return e.sm + e.lay->bvel + 6u * free_slot(e, b); }
NKB_DEV float* sm_bwinv(const Env& e, uint32_t b) { return e.sm + e.lay->bwinv + 6u * free_slot(e, b); }
NKB_DEV float* sm_aabb(const Env& e, uint32_t b) { return e.sm + e.lay->aabb + 6u * b; }
NKB_DEV uint32_t* sm_pairs(const Env& e) { return reinterpret_cast<uint32_t*>(e.sm + e.lay->pairs); }
NKB_DEV uint32_t* sm_ccount(const Env& e) { return reinterpret_cast<uint32_t*>(e.sm + e.lay->ccount); }
NKB_DEV float* sm_cpoint(const Env& e, uint32_t pt) { return e.sm + e.lay->cpoint + 3u * pt; }
NKB_DEV float* sm_cnormal(const Env& e, uint32_t pt) { return e.sm + e.lay->cnormal + 3u * pt; }
NKB_DEV float* sm_cdepth(const Env& e) { return e.sm + e.lay->cdepth; }
NKB_DEV uint32_t* sm_cfeat(const Env& e, uint32_t pt) { return reinterpret_cast<uint32_t*>(e.sm + e.lay->cfeat) + 2u * pt; }

// R diag(d) R^T with R from pose.rotation * inertial.rotation (ops/rigid_types.cuh:18-23)
NKB_DEV void world_inv_inertia(Q4 pose_q, Q4 inertial_q, V3 inv_i, float* out) {
    const M3 R = m3_from_quat(qmul(pose_q, inertial_q));
    const int ia[6] = {0, 1, 2, 0, 0, 1}, ib[6] = {0, 1, 2, 1, 2, 2};
    const float d[3] = {inv_i.x, inv_i.y, inv_i.z};
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < 3; ++c) s += R.m[ia[k] * 3 + c] * d[c] * R.m[ib[k] * 3 + c];
        out[k] = s;
    }
}

// Poses and velocities of every collidable row into shared memory; free bodies take their gravity kick.
NKB_DEV void stage_bodies(Env& e, bool kick) {
    const TemplateView& t = *e.t;
    const V3 g = mk3(t.cfg.gravity[0], t.cfg.gravity[1], t.cfg.gravity[2]);
    for (uint32_t b = e.lane; b < t.B; b += 32u) {
        const uint32_t link = __ldg(t.body_to_link + b);
        float* bp = sm_bpose(e, b);
        float* bv = sm_bvel(e, b);
        const size_t gb = (size_t)e.env * t.B + b;
        if (link != kNoLink) {
            const float* lp = sm_pose(e, link);
            if (__ldg(t.body_geom_kind + b) != 0u) {
                const Q4 pq = ldq(lp + 3);
                st3(bp, ld3(lp) + qrot(pq, ld3(t.body_geom_pos + 3u * b)));
                stq(bp + 3, qmul(pq, ldq(t.body_geom_quat + 4u * b)));
            } else {
#pragma unroll
                for (int k = 0; k < 7; ++k) bp[k] = lp[k];
            }
#pragma unroll
            for (int k = 0; k < 6; ++k) bv[k] = 0.f;
        } else {
            const float* gp = e.s->body_pose + gb * 7u;
#pragma unroll
            for (int k = 0; k < 7; ++k) bp[k] = gp[k];
            V3 lv = ld3(e.s->body_linvel + gb * 3u);
            const V3 av = ld3(e.s->body_angvel + gb * 3u);
            const bool dynamic = __ldg(t.inv_mass + b) > 0.f;
            if (kick && dynamic) lv = lv + g * t.cfg.dt;
            if (dynamic) { st3(bv, lv); st3(bv + 3, av); }
            else { st3(bv, mk3(0.f, 0.f, 0.f)); st3(bv + 3, mk3(0.f, 0.f, 0.f)); }      // static rows share the zero slot
        }
        float* w = sm_bwinv(e, b);
        if (__ldg(t.inv_mass + b) > 0.f) world_inv_inertia(ldq(bp + 3), ldq(t.inertial_quat + 4u * b), ld3(t.inv_inertia + 3u * b), w);
        else {
#pragma unroll
            for (int k = 0; k < 6; ++k) w[k] = 0.f;
        }
    }
    __syncwarp();
}

NKB_DEV V3 rot_abs(Q4 q, V3 v) {
    const V3 cx = qrot_raw(q, mk3(1.f, 0.f, 0.f)), cy = qrot_raw(q, mk3(0.f, 1.f, 0.f)), cz = qrot_raw(q, mk3(0.f, 0.f, 1.f));
    return mk3(fabsf(cx.x) * v.x + fabsf(cy.x) * v.y + fabsf(cz.x) * v.z, fabsf(cx.y) * v.x + fabsf(cy.y) * v.y + fabsf(cz.y) * v.z,
               fabsf(cx.z) * v.x + fabsf(cy.z) * v.y + fabsf(cz.z) * v.z);
}
NKB_DEV float query_reach(const Config& c) { return fmaxf(0.02f, 2.0f * (2.0f * 0.0f + c.contact_margin)); }
NKB_DEV float motion_radius(float base, float dt, float sa, float sb) { return base + dt * (sa + sb) * (2.0f / 0.9f); }

NKB_DEV void stage_aabbs(Env& e) {
    const TemplateView& t = *e.t;
    const float margin = fmaxf(t.cfg.contact_margin, 0.0005f), reach = query_reach(t.cfg);
    for (uint32_t b = e.lane; b < t.B; b += 32u) {
        const float* bp = sm_bpose(e, b);
        const float* p = t.shape_params + 4u * b;
        const V3 c = ld3(bp);
        const Q4 q = ldq(bp + 3);
        V3 he = mk3(0.f, 0.f, 0.f);
        float* out = sm_aabb(e, b);
        const uint32_t kind = __ldg(t.shape_kind + b);
        if (kind == kPlane) {
            out[0] = out[1] = out[2] = -FLT_MAX; out[3] = out[4] = out[5] = FLT_MAX;
            continue;
        }
        if (kind == kSphere) he = mk3(p[0], p[0], p[0]);
        else if (kind == kCapsule) he = rot_abs(q, mk3(p[0], p[0], p[0] + p[1]));
        else if (kind == kBox) he = rot_abs(q, mk3(p[0], p[1], p[2]));
        else { out[0] = out[1] = out[2] = FLT_MAX; out[3] = out[4] = out[5] = -FLT_MAX; continue; }
        const float radius = sqrtf(dot(he, he)) + 0.0f;
        const float* bv = sm_bvel(e, b);
        const float speed = fmaxf(0.0f, len3(ld3(bv)) + len3(ld3(bv + 3)) * radius);
        const float mm = fmaxf(margin, fminf(motion_radius(margin, t.cfg.dt, speed, 0.0f), reach));
        out[0] = c.x - he.x - mm; out[1] = c.y - he.y - mm; out[2] = c.z - he.z - mm;
        out[3] = c.x + he.x + mm; out[4] = c.y + he.y + mm; out[5] = c.z + he.z + mm;
    }
    __syncwarp();
}

// Candidate pairs in ascending (a, b) order: the admissible-pair table is walked 32 entries at a time and
// overlapping pairs are compacted in order, so the list needs no sort.  Returns the pair count.
NKB_DEV uint32_t stage_pairs(Env& e) {
    const TemplateView& t = *e.t;
    const uint32_t cap = t.cfg.max_pairs != 0u && t.cfg.max_pairs < t.cfg.max_contacts ? t.cfg.max_pairs : t.cfg.max_contacts;
    uint32_t count = 0u;
    uint32_t* pairs = sm_pairs(e);
    for (uint32_t base = 0u; base < t.n_adm; base += 32u) {
        const uint32_t k = base + e.lane;
        bool hit = false;
        uint32_t ab = 0u;
        if (k < t.n_adm) {
            ab = __ldg(t.adm_pairs + k);
            const float* A = sm_aabb(e, ab >> 16);
            const float* Bx = sm_aabb(e, ab & 0xffffu);
            hit = !(A[3] < Bx[0] || A[0] > Bx[3] || A[4] < Bx[1] || A[1] > Bx[4] || A[5] < Bx[2] || A[2] > Bx[5]);
        }
        const uint32_t mask = __ballot_sync(NKB_FULL, hit);
        const uint32_t at = count + __popc(mask & ((1u << e.lane) - 1u));
        if (hit) { if (at < cap) pairs[at] = ab; else e.status |= kStatusPairOverflow; }
        count += __popc(mask);
    }
    __syncwarp();
    return count < cap ? count : cap;
}

// ---- analytic manifolds ----
struct Frame { V3 cx, cy, cz, t; };
struct Prim { V3 he; float radius, hh; Frame f; };
struct Manifold { uint32_t count; V3 pos[4]; V3 n[4]; float pen[4]; uint32_t key[4]; };
struct Cand { V3 pos; float pen; uint32_t feat; };

NKB_DEV V3 f_l2w(const Frame& f, V3 l) {
    return mk3(f.cx.x * l.x + f.cy.x * l.y + f.cz.x * l.z + f.t.x, f.cx.y * l.x + f.cy.y * l.y + f.cz.y * l.z + f.t.y,
               f.cx.z * l.x + f.cy.z * l.y + f.cz.z * l.z + f.t.z);
}
NKB_DEV V3 f_w2l(const Frame& f, V3 w) { const V3 d = w - f.t; return mk3(dot(d, f.cx), dot(d, f.cy), dot(d, f.cz)); }
NKB_DEV V3 f_dir(const Frame& f, V3 l) {
    return mk3(f.cx.x * l.x + f.cy.x * l.y + f.cz.x * l.z, f.cx.y * l.x + f.cy.y * l.y + f.cz.y * l.z, f.cx.z * l.x + f.cy.z * l.y + f.cz.z * l.z);
}
NKB_DEV V3 f_axis(const Frame& f, int k) { return k == 0 ? f.cx : (k == 1 ? f.cy : f.cz); }
NKB_DEV V3 norm_or(V3 v, V3 fb) { const float l = len3(v); if (l < 1.0e-12f) return fb; return mk3(v.x / l, v.y / l, v.z / l); }
NKB_DEV void add_pt(Manifold& o, V3 pos, V3 n, float pen, uint32_t key) {
    if (o.count < 4u) { o.pos[o.count] = pos; o.n[o.count] = n; o.pen[o.count] = pen; o.key[o.count] = key; ++o.count; }
}

static __device__ __noinline__ void reduce_emit(Cand* c, int n, V3 normal, Manifold& o) {
    if (n <= 0) return;
    const int keep = n < 4 ? n : 4;
    for (int s = 0; s < keep; ++s) {
        int best = s;
        for (int i = s + 1; i < n; ++i)
            if (c[i].pen > c[best].pen || (c[i].pen == c[best].pen && c[i].feat < c[best].feat)) best = i;
        const Cand tmp = c[s]; c[s] = c[best]; c[best] = tmp;
    }
    for (int i = 1; i < keep; ++i) {
        const Cand key = c[i]; int j = i - 1;
        while (j >= 0 && c[j].feat > key.feat) { c[j + 1] = c[j]; --j; }
        c[j + 1] = key;
    }
    o.count = 0;
    for (int i = 0; i < keep; ++i) add_pt(o, c[i].pos, normal, c[i].pen, c[i].feat);
}

static __device__ __noinline__ void reduce_emit_spread(Cand* c, int n, V3 normal, Manifold& o) {
    o.count = 0;
    if (n <= 0) return;
    if (n <= 4) {
        for (int i = 1; i < n; ++i) {
            const Cand key = c[i]; int j = i - 1;
            while (j >= 0 && c[j].feat > key.feat) { c[j + 1] = c[j]; --j; }
            c[j + 1] = key;
        }
        for (int i = 0; i < n; ++i) add_pt(o, c[i].pos, normal, c[i].pen, c[i].feat);
        return;
    }
    int kept[4] = {0, 0, 0, 0};
    uint32_t used = 0u;
    int seed = 0;
    for (int i = 1; i < n; ++i) if (c[i].pen > c[seed].pen) seed = i;
    kept[0] = seed; used |= 1u << seed;
    for (int s = 1; s < 4; ++s) {
        int best = -1; float best_mind = -1.0f;
        for (int i = 0; i < n; ++i) {
            if ((used >> i) & 1u) continue;
            float mind = 3.4e38f;
            for (int q = 0; q < s; ++q) { const V3 d = c[i].pos - c[kept[q]].pos; const float dd = dot(d, d); if (dd < mind) mind = dd; }
            if (mind > best_mind) { best_mind = mind; best = i; }
        }
        if (best < 0) break;
        kept[s] = best; used |= 1u << best;
    }
    for (int i = 1; i < 4; ++i) {
        const int key = kept[i]; int j = i - 1;
        while (j >= 0 && c[kept[j]].feat > c[key].feat) { kept[j + 1] = kept[j]; --j; }
        kept[j + 1] = key;
    }
    for (int i = 0; i < 4; ++i) add_pt(o, c[kept[i]].pos, normal, c[kept[i]].pen, c[kept[i]].feat);
}

NKB_DEV void sphere_sphere(const Prim& a, const Prim& b, Manifold& o, float query) {
    const V3 delta = a.f.t - b.f.t;
    const float dist = len3(delta), pen = (a.radius + b.radius) - dist;
    if (pen <= -query) return;
    const V3 n = norm_or(delta, mk3(0.f, 1.f, 0.f));
    add_pt(o, b.f.t + n * (b.radius - 0.5f * pen), n, pen, 0u);
}
NKB_DEV bool surface_box(V3 he, V3 p, float& dist, V3& normal, V3& point) {
    if (!(he.x >= 0.f && he.y >= 0.f && he.z >= 0.f)) return false;
    const V3 cl = mk3(fmaxf(-he.x, fminf(p.x, he.x)), fmaxf(-he.y, fminf(p.y, he.y)), fmaxf(-he.z, fminf(p.z, he.z)));
    const V3 off = p - cl;
    const float len = sqrtf(dot(off, off));
    if (len > 0.f) { dist = len; normal = mk3(off.x / len, off.y / len, off.z / len); }
    else {
        const V3 d = mk3(fabsf(p.x) - he.x, fabsf(p.y) - he.y, fabsf(p.z) - he.z);
        if (d.x >= d.y && d.x >= d.z) { dist = d.x; normal = mk3(p.x < 0.f ? -1.f : 1.f, 0.f, 0.f); }
        else if (d.y >= d.z) { dist = d.y; normal = mk3(0.f, p.y < 0.f ? -1.f : 1.f, 0.f); }
        else { dist = d.z; normal = mk3(0.f, 0.f, p.z < 0.f ? -1.f : 1.f); }
    }
    point = p - normal * dist;
    return true;
}
NKB_DEV bool surface_capsule(float r, float hh, V3 p, float& dist, V3& normal, V3& point) {
    if (!(r >= 0.f) || !(hh >= 0.f)) return false;
    V3 off = p;
    off.z -= fmaxf(-hh, fminf(p.z, hh));
    const float len = sqrtf(dot(off, off));
    normal = mk3(1.f, 0.f, 0.f);
    if (len > 0.f) normal = mk3(off.x / len, off.y / len, off.z / len);
    dist = len - r;
    point = p - normal * dist;
    return true;
}
NKB_DEV void sphere_box(const Prim& s, const Prim& box, Manifold& o, float query) {
    float dist; V3 n, pt;
    if (!surface_box(box.he, f_w2l(box.f, s.f.t), dist, n, pt)) return;
    const float pen = s.radius - dist;
    if (pen <= -query) return;
    const V3 nw = f_dir(box.f, n);
    add_pt(o, f_l2w(box.f, pt) - nw * (0.5f * pen), nw, pen, 0u);
}
NKB_DEV void sphere_plane(const Prim& s, const Prim& pl, Manifold& o, float query) {
    const V3 n = norm_or(pl.f.cz, mk3(0.f, 0.f, 1.f));
    const float sd = dot(s.f.t - pl.f.t, n), pen = s.radius - sd;
    if (pen <= -query) return;
    add_pt(o, s.f.t - n * (s.radius - 0.5f * pen), n, pen, 0u);
}
NKB_DEV void box_plane(const Prim& box, const Prim& pl, Manifold& o, float query) {
    const V3 n = norm_or(pl.f.cz, mk3(0.f, 0.f, 1.f));
    Cand c[8]; int nc = 0;
    for (uint32_t k = 0; k < 8u; ++k) {
        const float sx = (k & 1u) ? 1.f : -1.f, sy = (k & 2u) ? 1.f : -1.f, sz = (k & 4u) ? 1.f : -1.f;
        const V3 cw = f_l2w(box.f, mk3(sx * box.he.x, sy * box.he.y, sz * box.he.z));
        const float sd = dot(cw - pl.f.t, n);
        if (sd < query) { c[nc].pos = cw - n * (0.5f * sd); c[nc].pen = -sd; c[nc].feat = k; ++nc; }
    }
    reduce_emit(c, nc, n, o);
}
NKB_DEV void capsule_plane(const Prim& cap, const Prim& pl, Manifold& o, float query) {
    const V3 n = norm_or(pl.f.cz, mk3(0.f, 0.f, 1.f));
    const V3 ends[2] = {cap.f.t + cap.f.cz * cap.hh, cap.f.t - cap.f.cz * cap.hh};
    Cand c[2]; int nc = 0;
    for (uint32_t k = 0; k < 2u; ++k) {
        const float sd = dot(ends[k] - pl.f.t, n) - cap.radius;
        if (sd < query) { c[nc].pos = ends[k] - n * (cap.radius + 0.5f * sd); c[nc].pen = -sd; c[nc].feat = k; ++nc; }
    }
    reduce_emit(c, nc, n, o);
}
NKB_DEV void capsule_sphere(const Prim& cap, const Prim& s, Manifold& o, float query) {
    float dist; V3 n, pt;
    if (!surface_capsule(cap.radius, cap.hh, f_w2l(cap.f, s.f.t), dist, n, pt)) return;
    const float pen = s.radius - dist;
    if (pen <= -query) return;
    const V3 nw = f_dir(cap.f, n) * -1.0f;
    add_pt(o, f_l2w(cap.f, pt) + nw * (0.5f * pen), nw, pen, 0u);
}
NKB_DEV float closest_seg_seg(V3 p1, V3 q1, V3 p2, V3 q2, V3& c1, V3& c2) {
    const V3 d1 = q1 - p1, d2 = q2 - p2, r = p1 - p2;
    const float a = dot(d1, d1), e = dot(d2, d2), f = dot(d2, r);
    float s = 0.f, t = 0.f;
    const float eps = 1.0e-12f;
    if (a <= eps && e <= eps) { s = t = 0.f; }
    else if (a <= eps) { s = 0.f; t = f / e; t = t < 0.f ? 0.f : (t > 1.f ? 1.f : t); }
    else {
        const float c = dot(d1, r);
        if (e <= eps) { t = 0.f; s = -c / a; s = s < 0.f ? 0.f : (s > 1.f ? 1.f : s); }
        else {
            const float b = dot(d1, d2), denom = a * e - b * b;
            if (denom > eps) { s = (b * f - c * e) / denom; s = s < 0.f ? 0.f : (s > 1.f ? 1.f : s); } else s = 0.f;
            t = (b * s + f) / e;
            if (t < 0.f) { t = 0.f; s = -c / a; s = s < 0.f ? 0.f : (s > 1.f ? 1.f : s); }
            else if (t > 1.f) { t = 1.f; s = (b - c) / a; s = s < 0.f ? 0.f : (s > 1.f ? 1.f : s); }
        }
    }
    c1 = p1 + d1 * s; c2 = p2 + d2 * t;
    const V3 dv = c1 - c2;
    return dot(dv, dv);
}
NKB_DEV void capsule_capsule(const Prim& a, const Prim& b, Manifold& o, float query) {
    const V3 axa = a.f.cz, axb = b.f.cz;
    V3 ca, cb;
    const float d2 = closest_seg_seg(a.f.t + axa * a.hh, a.f.t - axa * a.hh, b.f.t + axb * b.hh, b.f.t - axb * b.hh, ca, cb);
    const float dist = sqrtf(d2), pen = (a.radius + b.radius) - dist;
    if (pen <= -query) return;
    const V3 n = norm_or(ca - cb, norm_or(cross(axa, axb), mk3(0.f, 1.f, 0.f)));
    const V3 sa = ca - n * a.radius, sb = cb + n * b.radius;
    add_pt(o, (sa + sb) * 0.5f, n, pen, 0u);
}

struct ClipPoly { V3 v[8]; int count; };
NKB_DEV void poly_add(ClipPoly& p, V3 v) { if (p.count < 8) { p.v[p.count] = v; ++p.count; } }
static __device__ __noinline__ void clip_plane(const ClipPoly& in, V3 pp, V3 pn, ClipPoly& out) {
    out.count = 0;
    for (int i = 0; i < in.count; ++i) {
        const int j = (i + 1) % in.count;
        const V3 cur = in.v[i], nxt = in.v[j];
        const float dc = dot(cur - pp, pn), dn = dot(nxt - pp, pn);
        const bool ci = dc <= 0.f, ni = dn <= 0.f;
        if (ci) poly_add(out, cur);
        if (ci != ni) {
            const float tt = dc / (dc - dn);
            poly_add(out, mk3(cur.x + (nxt.x - cur.x) * tt, cur.y + (nxt.y - cur.y) * tt, cur.z + (nxt.z - cur.z) * tt));
        }
    }
}
NKB_DEV float fabs_dot(V3 a, V3 b) { const float d = dot(a, b); return d < 0.f ? -d : d; }

static __device__ __noinline__ void box_box(const Prim& A, const Prim& B, Manifold& o, float query) {
    const V3 ha = A.he, hb = B.he, dpos = B.f.t - A.f.t;
    const V3 ax[3] = {A.f.cx, A.f.cy, A.f.cz}, bx[3] = {B.f.cx, B.f.cy, B.f.cz};
    float AbsR[3][3];
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) { const float r = dot(ax[i], bx[j]); AbsR[i][j] = (r < 0.f ? -r : r) + 1.0e-6f; }
    const float ea[3] = {ha.x, ha.y, ha.z}, eb[3] = {hb.x, hb.y, hb.z};
    const float dA[3] = {dot(dpos, ax[0]), dot(dpos, ax[1]), dot(dpos, ax[2])};
    float min_pen = 3.4e38f; int best_axis = -1; V3 best_n = mk3(0.f, 1.f, 0.f);
    const float bias = 1.0e-5f;
    for (int i = 0; i < 3; ++i) {
        const float ra = ea[i], rb = eb[0] * AbsR[i][0] + eb[1] * AbsR[i][1] + eb[2] * AbsR[i][2];
        const float s = dA[i] < 0.f ? -dA[i] : dA[i], pen = (ra + rb) - s;
        if (pen <= -query) return;
        if (pen < min_pen - bias) { min_pen = pen; best_axis = i; best_n = dA[i] < 0.f ? -ax[i] : ax[i]; }
    }
    for (int j = 0; j < 3; ++j) {
        const float ra = ea[0] * AbsR[0][j] + ea[1] * AbsR[1][j] + ea[2] * AbsR[2][j], rb = eb[j];
        const float dB = dot(dpos, bx[j]), s = dB < 0.f ? -dB : dB, pen = (ra + rb) - s;
        if (pen <= -query) return;
        if (pen < min_pen - bias) { min_pen = pen; best_axis = 3 + j; best_n = dB < 0.f ? -bx[j] : bx[j]; }
    }
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) {
        V3 Lx = cross(ax[i], bx[j]);
        const float ll = len3(Lx);
        if (ll < 1.0e-6f) continue;
        Lx = mk3(Lx.x / ll, Lx.y / ll, Lx.z / ll);
        const float ra = ea[0] * fabs_dot(ax[0], Lx) + ea[1] * fabs_dot(ax[1], Lx) + ea[2] * fabs_dot(ax[2], Lx);
        const float rb = eb[0] * fabs_dot(bx[0], Lx) + eb[1] * fabs_dot(bx[1], Lx) + eb[2] * fabs_dot(bx[2], Lx);
        const float s = dot(dpos, Lx), sa = s < 0.f ? -s : s, pen = (ra + rb) - sa;
        if (pen <= -query) return;
        if (pen < min_pen - bias) { min_pen = pen; best_axis = 6 + i * 3 + j; best_n = s < 0.f ? -Lx : Lx; }
    }
    if (best_axis < 0) return;
    if (best_axis >= 6) {
        const int i = (best_axis - 6) / 3, j = (best_axis - 6) % 3;
        V3 pa = A.f.t, pb = B.f.t;
        for (int k = 0; k < 3; ++k) { if (k == i) continue; const float sg = dot(ax[k], best_n) >= 0.f ? 1.f : -1.f; pa = pa + ax[k] * (sg * ea[k]); }
        for (int k = 0; k < 3; ++k) { if (k == j) continue; const float sg = dot(bx[k], best_n) >= 0.f ? -1.f : 1.f; pb = pb + bx[k] * (sg * eb[k]); }
        const V3 ed = ax[i], fd = bx[j], r = pa - pb;
        const float aa = 1.f, bb = dot(ed, fd), cc = 1.f, dd = dot(ed, r), ee = dot(fd, r), denom = aa * cc - bb * bb;
        float sN = 0.f, tN = 0.f;
        if (denom > 1.0e-9f) { sN = (bb * ee - cc * dd) / denom; tN = (aa * ee - bb * dd) / denom; }
        const float sC = sN < -ea[i] ? -ea[i] : (sN > ea[i] ? ea[i] : sN), tC = tN < -eb[j] ? -eb[j] : (tN > eb[j] ? eb[j] : tN);
        const V3 ca = pa + ed * sC, cb = pb + fd * tC;
        add_pt(o, (ca + cb) * 0.5f, best_n, min_pen, 0xE0000000u | ((uint32_t)i << 4) | (uint32_t)j);
        return;
    }
    const bool ref_is_A = best_axis < 3;
    const int ref_axis = ref_is_A ? best_axis : best_axis - 3;
    const Frame& Rf = ref_is_A ? A.f : B.f;
    const Frame& If = ref_is_A ? B.f : A.f;
    const V3 rhe = ref_is_A ? ha : hb, ihe = ref_is_A ? hb : ha;
    V3 refN = f_axis(Rf, ref_axis);
    if (dot(If.t - Rf.t, refN) < 0.f) refN = -refN;
    int inc_axis = 0; float best_dot = 3.4e38f, inc_sign = 1.f;
    for (int k = 0; k < 3; ++k) {
        const float d = dot(f_axis(If, k), refN), ad = d < 0.f ? -d : d;
        if (-ad < best_dot) { best_dot = -ad; inc_axis = k; inc_sign = d < 0.f ? 1.f : -1.f; }
    }
    const int iu = (inc_axis + 1) % 3, iv = (inc_axis + 2) % 3;
    const V3 ifc = If.t + f_axis(If, inc_axis) * (inc_sign * comp(ihe, inc_axis));
    const V3 iuw = f_axis(If, iu), ivw = f_axis(If, iv);
    const float iue = comp(ihe, iu), ive = comp(ihe, iv);
    ClipPoly pa, pb;
    pa.count = 0;
    const float su[4] = {-1.f, 1.f, 1.f, -1.f}, sv[4] = {-1.f, -1.f, 1.f, 1.f};
    for (int k = 0; k < 4; ++k) poly_add(pa, ifc + iuw * (su[k] * iue) + ivw * (sv[k] * ive));
    const int ru = (ref_axis + 1) % 3, rv = (ref_axis + 2) % 3;
    const V3 ruw = f_axis(Rf, ru), rvw = f_axis(Rf, rv);
    const float rue = comp(rhe, ru), rve = comp(rhe, rv);
    const V3 rfc = Rf.t + refN * comp(rhe, ref_axis);
    clip_plane(pa, rfc + ruw * rue, ruw, pb);
    clip_plane(pb, rfc - ruw * rue, -ruw, pa);
    clip_plane(pa, rfc + rvw * rve, rvw, pb);
    clip_plane(pb, rfc - rvw * rve, -rvw, pa);
    Cand c[8]; int nc = 0;
    for (int k = 0; k < pa.count; ++k) {
        const float depth = dot(rfc - pa.v[k], refN);
        if (depth >= -query) {
            const V3 onref = pa.v[k] + refN * depth;
            c[nc].pos = (pa.v[k] + onref) * 0.5f; c[nc].pen = depth; c[nc].feat = (uint32_t)k; ++nc;
        }
    }
    const V3 nA = ref_is_A ? -refN : refN;
    if (nc == 0) { add_pt(o, ifc + refN * (min_pen * 0.5f), nA, min_pen, (uint32_t)inc_axis << 4); return; }
    reduce_emit_spread(c, nc, nA, o);
}

NKB_DEV void primitive_pair(uint32_t ka, const Prim& a, uint32_t kb, const Prim& b, float query, Manifold& o) {
    o.count = 0;
    if (ka == kSphere && kb == kSphere) { sphere_sphere(a, b, o, query); return; }
    if (ka == kSphere && kb == kBox) { sphere_box(a, b, o, query); return; }
    if (ka == kSphere && kb == kPlane) { sphere_plane(a, b, o, query); return; }
    if (ka == kBox && kb == kPlane) { box_plane(a, b, o, query); return; }
    if (ka == kBox && kb == kBox) { box_box(a, b, o, query); return; }
    if (ka == kCapsule && kb == kPlane) { capsule_plane(a, b, o, query); return; }
    if (ka == kCapsule && kb == kSphere) { capsule_sphere(a, b, o, query); return; }
    if (ka == kCapsule && kb == kCapsule) { capsule_capsule(a, b, o, query); return; }
    bool done = true;
    if (ka == kBox && kb == kSphere) sphere_box(b, a, o, query);
    else if (ka == kPlane && kb == kSphere) sphere_plane(b, a, o, query);
    else if (ka == kPlane && kb == kBox) box_plane(b, a, o, query);
    else if (ka == kPlane && kb == kCapsule) capsule_plane(b, a, o, query);
    else if (ka == kSphere && kb == kCapsule) capsule_sphere(b, a, o, query);
    else done = false;
    if (done) for (uint32_t i = 0; i < o.count; ++i) o.n[i] = -o.n[i];
}

NKB_DEV Prim make_prim(const Env& e, uint32_t b) {
    Prim p;
    const float* bp = sm_bpose(e, b);
    const Q4 q = ldq(bp + 3);
    p.f.cx = qrot_raw(q, mk3(1.f, 0.f, 0.f)); p.f.cy = qrot_raw(q, mk3(0.f, 1.f, 0.f)); p.f.cz = qrot_raw(q, mk3(0.f, 0.f, 1.f));
    p.f.t = ld3(bp);
    const float* s = e.t->shape_params + 4u * b;
    p.radius = s[0]; p.hh = s[1]; p.he = mk3(s[0], s[1], s[2]);
    return p;
}
NKB_DEV float body_speed(const Env& e, uint32_t b) {
    const V3 c = ld3(sm_bpose(e, b));
    const float* ab = sm_aabb(e, b);
    const V3 lo = ld3(ab) - c, hi = ld3(ab + 3) - c;
    const V3 ext = mk3(fmaxf(fabsf(lo.x), fabsf(hi.x)), fmaxf(fabsf(lo.y), fabsf(hi.y)), fmaxf(fabsf(lo.z), fabsf(hi.z)));
    const V3 w = ld3(sm_bvel(e, b) + 3);
    return fmaxf(0.0f, len3(ld3(sm_bvel(e, b))) + sqrtf(dot(w, w) * dot(ext, ext)));
}
NKB_DEV unsigned long long hash_word(unsigned long long h, unsigned long long w) { h ^= w; h *= 1099511628211ull; return h; }
NKB_DEV int quantize(float v) { const float s = v * 4096.0f; const float r = s >= 0.f ? s + 0.5f : s - 0.5f; return (int)r; }
NKB_DEV unsigned long long feature_token(uint32_t feature, V3 p) {
    if (feature != 0xffffffffu) return 0x8000000000000000ull | (unsigned long long)feature;
    unsigned long long h = 1469598103934665603ull;
    h = hash_word(h, (uint32_t)quantize(p.x)); h = hash_word(h, (uint32_t)quantize(p.y)); h = hash_word(h, (uint32_t)quantize(p.z));
    return h & 0x7fffffffffffffffull;
}
NKB_DEV V3 inv_xf_point(const float* pose, V3 w) {
    const V3 v = w - ld3(pose);
    const Q4 q = ldq(pose + 3);
    return qrot_raw(mkq(q.w, -q.x, -q.y, -q.z), v);
}

// One lane per candidate slot: analytic manifold, speculative depth (+ separation shell), contact identity.
NKB_DEV void stage_narrowphase(Env& e, uint32_t pair_count) {
    const TemplateView& t = *e.t;
    const float separation = fmaxf(t.cfg.contact_margin, 0.0005f), reach = query_reach(t.cfg);
    const uint32_t S = t.slot_cap;            // slots past the admissible-pair count can never fill and have no storage
    uint32_t* cc = sm_ccount(e);
    for (uint32_t s = e.lane; s < S; s += 32u) {
        uint32_t count = 0u;
        if (s < pair_count) {
            const uint32_t ab = sm_pairs(e)[s], a = ab >> 16, b = ab & 0xffffu;
            const Prim pa = make_prim(e, a), pb = make_prim(e, b);
            const float query = fmaxf(separation, fminf(motion_radius(2.0f * separation, t.cfg.dt, body_speed(e, a), body_speed(e, b)), reach));
            Manifold mf;
            primitive_pair(__ldg(t.shape_kind + a), pa, __ldg(t.shape_kind + b), pb, query, mf);
            count = mf.count;
            for (uint32_t i = 0; i < mf.count; ++i) {
                const uint32_t at = s * 4u + i;
                st3(sm_cpoint(e, at), mf.pos[i]);
                st3(sm_cnormal(e, at), mf.n[i]);
                sm_cdepth(e)[at] = mf.pen[i] + separation;
                const V3 la = inv_xf_point(sm_bpose(e, a), mf.pos[i]), lb = inv_xf_point(sm_bpose(e, b), mf.pos[i]);
                const uint32_t feature = mf.key[i] == 0u ? 0xffffffffu : mf.key[i];
                unsigned long long h = 1469598103934665603ull;
                h = hash_word(h, feature_token(feature, la));
                h = hash_word(h, feature_token(feature, lb));
                h = hash_word(h, i); h = hash_word(h, 0u); h = hash_word(h, 0u);
                uint32_t* f = sm_cfeat(e, at);
                f[0] = (uint32_t)h; f[1] = (uint32_t)(h >> 32);
            }
        }
        cc[s] = count;
    }
    __syncwarp();
}

// Contact read-out to global memory (pairs, counts, points, normals, depths).
NKB_DEV void stage_store_contacts(Env& e, uint32_t pair_count) {
    const TemplateView& t = *e.t;
    const uint32_t S = t.cfg.max_contacts;
    if (e.s->pair_count == nullptr || S == 0u) return;
    if (e.lane == 0u) e.s->pair_count[e.env] = pair_count;
    for (uint32_t s = e.lane; s < S; s += 32u) {
        const size_t gs = (size_t)e.env * S + s;
        const uint32_t ab = s < pair_count ? sm_pairs(e)[s] : 0u;
        e.s->pairs[gs * 2u] = ab >> 16; e.s->pairs[gs * 2u + 1u] = ab & 0xffffu;
        const uint32_t n = s < t.slot_cap ? sm_ccount(e)[s] : 0u;
        e.s->contact_count[gs] = n;
        for (uint32_t i = 0; i < 4u; ++i) {
            const bool live = i < n;
            const uint32_t at = s * 4u + i;
            const V3 p = live ? ld3(sm_cpoint(e, at)) : mk3(0.f, 0.f, 0.f), nn = live ? ld3(sm_cnormal(e, at)) : mk3(0.f, 0.f, 0.f);
            st3(e.s->contact_point + (gs * 4u + i) * 3u, p);
            st3(e.s->contact_normal + (gs * 4u + i) * 3u, nn);
            e.s->contact_depth[gs * 4u + i] = live ? sm_cdepth(e)[at] : 0.f;
        }
    }
}

}  // namespace nkb
