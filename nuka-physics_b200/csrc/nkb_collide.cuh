// Warp-per-env collision stages: collidable poses, free-body velocity kick, inflated AABBs, candidate pairs from the
// admissible-pair table, and the contact read-out.  Quantities follow the reference's ops/sync_body_pose.cu:24-50,
// ops/articulation.cu:1019-1051, ops/broadphase.cu:173-270 and :276-474 (pair predicate).  The tree broadphase is in
// nkb_lbvh.cuh, the contact manifolds in nkb_manifold.cuh.
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
        else if (kind == kCylinder) {
            // exact: along each world axis hh |a_i| + r sqrt(1 - a_i^2), a the cylinder's axis (ops/broadphase.cu:199-208)
            const V3 qv = mk3(q.x, q.y, q.z), ez = mk3(0.f, 0.f, 1.f);
            const V3 tz = cross(qv, ez) * 2.0f;
            const V3 a = ez + tz * q.w + cross(qv, tz);
            he = mk3(p[1] * fabsf(a.x) + p[0] * sqrtf(fmaxf(0.0f, 1.0f - a.x * a.x)),
                     p[1] * fabsf(a.y) + p[0] * sqrtf(fmaxf(0.0f, 1.0f - a.y * a.y)),
                     p[1] * fabsf(a.z) + p[0] * sqrtf(fmaxf(0.0f, 1.0f - a.z * a.z)));
        }
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
