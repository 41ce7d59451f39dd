// Warp-cooperative analytic narrowphase of one env.  Candidate slots are sorted by the work their shape pair needs and
// the warp's lanes are dealt out accordingly:
//   round pairs (a sphere or capsule against anything but a box-box / box-plane manifold)   1 lane per pair, registers only
//   box on plane                                                                              8 lanes per pair, lane = box corner
//   cylinder on plane                                                                        16 lanes per pair, lane = rim point
//   box on box                                                                               16 lanes per pair, lane = separating-axis
//                                                                                            candidate, then lane = polygon vertex
// Selections that a serial code does with arrays and loops (deepest four corners, farthest-point spread, polygon clipping)
// are done with ranks, ballots and sub-warp shuffles; the clipped polygon passes through a few words of shared memory per
// group, nothing lives in local memory.  What is computed per pair kind - contact points, normals, depths, the order of
// points and their feature keys - is the reference's analytic manifold (src/collision/analytical_manifold.hpp:416-966,
// dispatched by ops/narrowphase_prims.cu:181-366): separating axes are taken in its order with its 1e-5 preference for
// earlier axes, polygons are clipped edge by edge in its side order, at most four points survive by its rules (deepest
// first with ties to the lower feature for corners; deepest seed then farthest-from-kept for clipped faces), and points
// come out in ascending feature order.
#pragma once
#include "nkb_collide.cuh"

namespace nkb {

// World frame of one collidable row: axes cx, cy, cz then origin (12 words), cached once per step for the groups to share.
struct BodyFrame { V3 cx, cy, cz, t; };

// What the pair handlers touch, as plain pointers passed by value: the handlers are real functions (one copy each in the
// kernel), and a reference to the warp's Env would force that whole structure into local memory around every call.
struct PairCtx {
    float* sm;
    const SmemLayout* lay;
    const TemplateView* t;
    uint32_t lane;
    float separation;
    uint32_t stage_shift;       // words from the first warp's polygon staging areas to this warp's (team mode)
};
NKB_DEV PairCtx pair_ctx(const Env& e, float separation) {
    PairCtx c;
    c.sm = e.sm; c.lay = e.lay; c.t = e.t; c.lane = e.lane; c.separation = separation; c.stage_shift = 0u;
    return c;
}
NKB_DEV float* ctx_frames(const PairCtx& c) { return c.sm + c.lay->heads; }                 // 12 B words
NKB_DEV float* ctx_clip_stage(const PairCtx& c, uint32_t group) { return c.sm + c.lay->heads + 12u * c.t->B + c.stage_shift + 32u * group; }   // 2 x 32 words
NKB_DEV const float* ctx_pose(const PairCtx& c, uint32_t b) { return c.sm + c.lay->bpose + 7u * b; }
NKB_DEV const float* ctx_shape(const PairCtx& c, uint32_t b) { return c.t->shape_params + 4u * b; }
NKB_DEV uint32_t* ctx_count(const PairCtx& c) { return reinterpret_cast<uint32_t*>(c.sm + c.lay->ccount); }
// axis k (0-2) or origin (k = 3) of body b's cached world frame
NKB_DEV V3 frame_vec(const PairCtx& c, uint32_t b, int k) { return ld3(ctx_frames(c) + 12u * b + 3u * (uint32_t)k); }

NKB_DEV BodyFrame load_frame(const PairCtx& c, uint32_t b) {
    const float* f = ctx_frames(c) + 12u * b;
    BodyFrame r;
    r.cx = ld3(f); r.cy = ld3(f + 3); r.cz = ld3(f + 6); r.t = ld3(f + 9);
    return r;
}
NKB_DEV V3 to_world(const BodyFrame& f, V3 l) {
    return mk3(f.cx.x * l.x + f.cy.x * l.y + f.cz.x * l.z + f.t.x, f.cx.y * l.x + f.cy.y * l.y + f.cz.y * l.z + f.t.y,
               f.cx.z * l.x + f.cy.z * l.y + f.cz.z * l.z + f.t.z);
}
NKB_DEV V3 dir_to_world(const BodyFrame& f, V3 l) {
    return mk3(f.cx.x * l.x + f.cy.x * l.y + f.cz.x * l.z, f.cx.y * l.x + f.cy.y * l.y + f.cz.y * l.z, f.cx.z * l.x + f.cy.z * l.y + f.cz.z * l.z);
}
NKB_DEV V3 to_local(const BodyFrame& f, V3 w) { const V3 d = w - f.t; return mk3(dot(d, f.cx), dot(d, f.cy), dot(d, f.cz)); }
NKB_DEV V3 frame_axis(const BodyFrame& f, int k) { return k == 0 ? f.cx : (k == 1 ? f.cy : f.cz); }
NKB_DEV V3 unit_or(V3 v, V3 fallback) { const float l = len3(v); return l < 1.0e-12f ? fallback : mk3(v.x / l, v.y / l, v.z / l); }

NKB_DEV float body_speed(const Env& e, uint32_t b) {
    const V3 c = ld3(sm_bpose(e, b));
    const float* ab = sm_aabb(e, b);
    const V3 lo = ld3(ab) - c, hi = ld3(ab + 3) - c;
    const V3 ext = mk3(fmaxf(fabsf(lo.x), fabsf(hi.x)), fmaxf(fabsf(lo.y), fabsf(hi.y)), fmaxf(fabsf(lo.z), fabsf(hi.z)));
    const V3 w = ld3(sm_bvel(e, b) + 3);
    return fmaxf(0.0f, len3(ld3(sm_bvel(e, b))) + sqrtf(dot(w, w) * dot(ext, ext)));
}

// ---- contact identity (src/nk/contact/contact_identity.hpp:118-160): a stable feature names the point; without one the
// ---- points' quantised body-local positions do ----
NKB_DEV unsigned long long fnv_step(unsigned long long h, unsigned long long w) { h ^= w; h *= 1099511628211ull; return h; }
NKB_DEV int bin4096(float v) { const float s = v * 4096.0f; return (int)(s >= 0.f ? s + 0.5f : s - 0.5f); }
NKB_DEV unsigned long long side_token(uint32_t feature, const float* pose, V3 world_point) {
    if (feature != 0xffffffffu) return 0x8000000000000000ull | (unsigned long long)feature;
    const Q4 q = ldq(pose + 3);
    const V3 p = qrot_raw(mkq(q.w, -q.x, -q.y, -q.z), world_point - ld3(pose));
    unsigned long long h = 1469598103934665603ull;
    h = fnv_step(h, (uint32_t)bin4096(p.x)); h = fnv_step(h, (uint32_t)bin4096(p.y)); h = fnv_step(h, (uint32_t)bin4096(p.z));
    return h & 0x7fffffffffffffffull;
}

// Stores point `index` of slot `slot`: position, normal, depth with the separation shell, identity words.  One copy in
// the kernel (it is reached from every pair class).
static __device__ __noinline__ void write_point(PairCtx c, uint32_t slot, uint32_t index, uint32_t a, uint32_t b, V3 pos, V3 normal, float pen, uint32_t key) {
    const uint32_t at = slot * 4u + index;
    st3(c.sm + c.lay->cpoint + 3u * at, pos);
    st3(c.sm + c.lay->cnormal + 3u * at, normal);
    c.sm[c.lay->cdepth + at] = pen + c.separation;
    const uint32_t feature = key == 0u ? 0xffffffffu : key;
    unsigned long long h = 1469598103934665603ull;
    h = fnv_step(h, side_token(feature, ctx_pose(c, a), pos));
    h = fnv_step(h, side_token(feature, ctx_pose(c, b), pos));
    h = fnv_step(h, index); h = fnv_step(h, 0u); h = fnv_step(h, 0u);
    uint32_t* f = reinterpret_cast<uint32_t*>(c.sm + c.lay->cfeat) + 2u * at;
    f[0] = (uint32_t)h; f[1] = (uint32_t)(h >> 32);
}

// ---- round pairs: one lane, at most two points, all in registers ----
struct RoundPoints { uint32_t count; V3 pos[2]; V3 normal; float pen[2]; uint32_t key[2]; };

// closest points of two segments (Ericson's clamped solve), squared distance returned
NKB_DEV float segment_closest(V3 p1, V3 q1, V3 p2, V3 q2, V3& c1, V3& c2) {
    const V3 d1 = q1 - p1, d2 = q2 - p2, r = p1 - p2;
    const float a = dot(d1, d1), e = dot(d2, d2), f = dot(d2, r);
    const float tiny = 1.0e-12f;
    float s = 0.f, t = 0.f;
    auto unit_clamp = [](float v) { return v < 0.f ? 0.f : (v > 1.f ? 1.f : v); };
    if (a <= tiny && e <= tiny) { s = t = 0.f; }
    else if (a <= tiny) { t = unit_clamp(f / e); }
    else {
        const float c = dot(d1, r);
        if (e <= tiny) { s = unit_clamp(-c / a); }
        else {
            const float b = dot(d1, d2), denom = a * e - b * b;
            s = denom > tiny ? unit_clamp((b * f - c * e) / denom) : 0.f;
            t = (b * s + f) / e;
            if (t < 0.f) { t = 0.f; s = unit_clamp(-c / a); }
            else if (t > 1.f) { t = 1.f; s = unit_clamp((b - c) / a); }
        }
    }
    c1 = p1 + d1 * s; c2 = p2 + d2 * t;
    const V3 gap = c1 - c2;
    return dot(gap, gap);
}

// Surface of a box (half extents he) seen from local point p: distance (negative inside), outward normal, surface point.
NKB_DEV bool box_surface(V3 he, V3 p, float& dist, V3& normal, V3& point) {
    if (!(he.x >= 0.f && he.y >= 0.f && he.z >= 0.f)) return false;
    const V3 inside = mk3(fmaxf(-he.x, fminf(p.x, he.x)), fmaxf(-he.y, fminf(p.y, he.y)), fmaxf(-he.z, fminf(p.z, he.z)));
    const V3 out = p - inside;
    const float len = sqrtf(dot(out, out));
    if (len > 0.f) { dist = len; normal = mk3(out.x / len, out.y / len, out.z / len); }
    else {      // inside: the face with the least depth, x before y before z on ties
        const V3 d = mk3(fabsf(p.x) - he.x, fabsf(p.y) - he.y, fabsf(p.z) - he.z);
        const int k = (d.x >= d.y && d.x >= d.z) ? 0 : (d.y >= d.z ? 1 : 2);
        dist = comp(d, k);
        normal = mk3(0.f, 0.f, 0.f);
        setc(normal, k, comp(p, k) < 0.f ? -1.f : 1.f);
    }
    point = p - normal * dist;
    return true;
}

// `ka`/`kb` in slot order; shapes' params pa, pb (radius / half height / half extents as the template stores them).
NKB_DEV void round_pair(uint32_t ka, const BodyFrame& fa, const float* pa, uint32_t kb, const BodyFrame& fb, const float* pb, float query,
                        RoundPoints& out) {
    out.count = 0u;
    out.key[0] = out.key[1] = 0u;
    // the handlers are written for (first, second) = (sphere|capsule, other); the mirrored orders swap and flip the normal
    const bool mirrored = (ka == kBox && kb == kSphere) || (ka == kPlane && (kb == kSphere || kb == kCapsule)) || (ka == kSphere && (kb == kCapsule || kb == kCylinder));
    const BodyFrame& f1 = mirrored ? fb : fa;
    const BodyFrame& f2 = mirrored ? fa : fb;
    const float* p1 = mirrored ? pb : pa;
    const float* p2 = mirrored ? pa : pb;
    const uint32_t k1 = mirrored ? kb : ka, k2 = mirrored ? ka : kb;
    const float r1 = p1[0];
    if (k1 == kSphere && k2 == kSphere) {
        const V3 delta = f1.t - f2.t;
        const float pen = (r1 + p2[0]) - len3(delta);
        if (pen > -query) {
            out.normal = unit_or(delta, mk3(0.f, 1.f, 0.f));
            out.pos[0] = f2.t + out.normal * (p2[0] - 0.5f * pen); out.pen[0] = pen; out.count = 1u;
        }
    } else if (k1 == kSphere && k2 == kBox) {
        float dist; V3 n, pt;
        if (box_surface(mk3(p2[0], p2[1], p2[2]), to_local(f2, f1.t), dist, n, pt)) {
            const float pen = r1 - dist;
            if (pen > -query) {
                out.normal = dir_to_world(f2, n);
                out.pos[0] = to_world(f2, pt) - out.normal * (0.5f * pen); out.pen[0] = pen; out.count = 1u;
            }
        }
    } else if (k1 == kSphere && k2 == kPlane) {
        const V3 n = unit_or(f2.cz, mk3(0.f, 0.f, 1.f));
        const float pen = r1 - dot(f1.t - f2.t, n);
        if (pen > -query) { out.normal = n; out.pos[0] = f1.t - n * (r1 - 0.5f * pen); out.pen[0] = pen; out.count = 1u; }
    } else if (k1 == kCapsule && k2 == kPlane) {
        // both cap centres against the plane; the deeper first when only... both kept (two slots), in end order
        const V3 n = unit_or(f2.cz, mk3(0.f, 0.f, 1.f));
        out.normal = n;
#pragma unroll
        for (int end = 0; end < 2; ++end) {
            const V3 c = end == 0 ? f1.t + f1.cz * p1[1] : f1.t - f1.cz * p1[1];
            const float sd = dot(c - f2.t, n) - r1;
            if (sd < query) {
                const uint32_t at = out.count++;
                out.pos[at] = c - n * (r1 + 0.5f * sd); out.pen[at] = -sd; out.key[at] = (uint32_t)end;
            }
        }
    } else if (k1 == kCapsule && k2 == kSphere) {
        if (r1 >= 0.f && p1[1] >= 0.f) {
            // the sphere centre in the capsule frame, against the capsule's core segment along local z
            const V3 p = to_local(f1, f2.t);
            V3 off = p;
            off.z -= fmaxf(-p1[1], fminf(p.z, p1[1]));
            const float len = sqrtf(dot(off, off));
            const V3 n = len > 0.f ? mk3(off.x / len, off.y / len, off.z / len) : mk3(1.f, 0.f, 0.f);
            const float dist = len - r1, pen = p2[0] - dist;
            if (pen > -query) {
                out.normal = dir_to_world(f1, n) * -1.0f;
                out.pos[0] = to_world(f1, p - n * dist) + out.normal * (0.5f * pen); out.pen[0] = pen; out.count = 1u;
            }
        }
    } else if (k1 == kCylinder && k2 == kSphere) {
        if (r1 >= 0.f && p1[1] >= 0.f) {
            // the sphere centre in the cylinder frame (axis along local z): outside both the side and a cap the rim is nearest,
            // else whichever of side and cap is closer to the surface; the feature (0 bottom cap, 1 side, 2 top cap, 3 bottom
            // rim, 4 top rim) is the point's key (collision/primitive_surface.hpp:89-114, analytical_manifold.hpp:818-834)
            const V3 p = to_local(f1, f2.t);
            const float rho = sqrtf(p.x * p.x + p.y * p.y);
            const V3 radial = rho > 0.f ? mk3(p.x / rho, p.y / rho, 0.f) : mk3(1.f, 0.f, 0.f);
            const V3 axial = mk3(0.f, 0.f, p.z < 0.f ? -1.f : 1.f);
            const float side = rho - r1, cap = fabsf(p.z) - p1[1];
            float dist; V3 n; uint32_t feature;
            if (side > 0.f && cap > 0.f) {
                dist = sqrtf(side * side + cap * cap);
                const V3 sum = radial * side + axial * cap;
                n = mk3(sum.x / dist, sum.y / dist, sum.z / dist);
                feature = p.z < 0.f ? 3u : 4u;
            } else if (side > cap) { dist = side; n = radial; feature = 1u; }
            else { dist = cap; n = axial; feature = p.z < 0.f ? 0u : 2u; }
            const float pen = p2[0] - dist;
            if (pen > -query) {
                out.normal = dir_to_world(f1, n) * -1.0f;
                out.pos[0] = to_world(f1, p - n * dist) + out.normal * (0.5f * pen); out.pen[0] = pen; out.key[0] = feature; out.count = 1u;
            }
        }
    } else if (k1 == kCapsule && k2 == kCapsule) {
        V3 c1, c2;
        const float d2 = segment_closest(f1.t + f1.cz * p1[1], f1.t - f1.cz * p1[1], f2.t + f2.cz * p2[1], f2.t - f2.cz * p2[1], c1, c2);
        const float pen = (r1 + p2[0]) - sqrtf(d2);
        if (pen > -query) {
            out.normal = unit_or(c1 - c2, unit_or(cross(f1.cz, f2.cz), mk3(0.f, 1.f, 0.f)));
            const V3 s1 = c1 - out.normal * r1, s2 = c2 + out.normal * p2[0];
            out.pos[0] = (s1 + s2) * 0.5f; out.pen[0] = pen; out.count = 1u;
        }
    }
    if (mirrored) out.normal = -out.normal;
    // a capsule end key of 0 is "no stable feature" like every other single point: only end 1 carries one
}

enum PairClass : uint32_t { kClassNone = 0u, kClassRound = 1u, kClassBoxPlane = 2u, kClassBoxBox = 3u, kClassCylinderPlane = 4u };
NKB_DEV uint32_t pair_class(uint32_t ka, uint32_t kb) {
    if (ka == kBox && kb == kBox) return kClassBoxBox;
    if ((ka == kCylinder && kb == kPlane) || (ka == kPlane && kb == kCylinder)) return kClassCylinderPlane;
    if ((ka == kCylinder && kb == kSphere) || (ka == kSphere && kb == kCylinder)) return kClassRound;
    if (ka == kCylinder || kb == kCylinder) return kClassNone;
    if ((ka == kBox && kb == kPlane) || (ka == kPlane && kb == kBox)) return kClassBoxPlane;
    const bool round_a = ka == kSphere || ka == kCapsule, round_b = kb == kSphere || kb == kCapsule;
    if ((round_a && (round_b || kb == kPlane)) || (round_b && ka == kPlane)) return kClassRound;
    if ((ka == kSphere && kb == kBox) || (ka == kBox && kb == kSphere)) return kClassRound;
    return kClassNone;          // capsule-box, plane-plane and cylinders against boxes, capsules or cylinders have no analytic manifold; the template check rejects them
}

// The lowest `want` set bits of `mask`: lane index of the g-th (g < want), or 32.
NKB_DEV uint32_t nth_set_bit(uint32_t mask, uint32_t g) {
    for (uint32_t k = 0u; k < g; ++k) mask &= mask - 1u;
    return mask != 0u ? (uint32_t)__ffs(mask) - 1u : 32u;
}

// ---- box on plane: 8 lanes, lane = corner; the four deepest corners survive (ties to the lower corner id) and come out in
// ---- corner order ----
static __device__ __noinline__ void box_plane_group(PairCtx c, bool active, uint32_t slot, uint32_t a, uint32_t b, bool box_first, float query) {
    const uint32_t lane = c.lane, corner = lane & 7u, gbase = lane & ~7u;
    const uint32_t box = box_first ? a : b, plane = box_first ? b : a;
    const BodyFrame fb = load_frame(c, box), fp = load_frame(c, plane);
    const float* he = ctx_shape(c, box);
    const V3 n = unit_or(fp.cz, mk3(0.f, 0.f, 1.f));
    const V3 cw = to_world(fb, mk3((corner & 1u) ? he[0] : -he[0], (corner & 2u) ? he[1] : -he[1], (corner & 4u) ? he[2] : -he[2]));
    const float sd = dot(cw - fp.t, n);
    const bool touching = active && sd < query;
    const float pen = -sd;
    // rank among the touching corners by (depth descending, corner ascending)
    uint32_t rank = 0u;
#pragma unroll
    for (uint32_t k = 0u; k < 8u; ++k) {
        const float other = __shfl_sync(NKB_FULL, pen, gbase + k);
        const bool other_touching = __shfl_sync(NKB_FULL, (int)touching, gbase + k) != 0;
        if (other_touching && (other > pen || (other == pen && k < corner))) ++rank;
    }
    const bool kept = touching && rank < 4u;
    const uint32_t kept_mask = (__ballot_sync(NKB_FULL, kept) >> gbase) & 0xffu;
    if (kept) write_point(c, slot, __popc(kept_mask & ((1u << corner) - 1u)), a, b, cw - n * (0.5f * sd), box_first ? n : -n, pen, corner);
    if (active && corner == 0u) ctx_count(c)[slot] = __popc(kept_mask);
}

// ---- cylinder on plane: 16 lanes, lane = candidate point in the reference's order (analytical_manifold.hpp:780-816).  A cap
// ---- that faces the plane (|axis . n| >= 0.95) contributes its deepest rim point and the eight points of its octagon
// ---- (lanes 0-8 of the lower cap); otherwise each cap contributes its deepest rim point (lanes 0, 1).  Up to four survive:
// ---- all of them when at most four touch, else the deepest and then three times the one farthest from those kept (lowest
// ---- lane on ties); they come out in feature order, which is lane order. ----
static __device__ __noinline__ void cylinder_plane_group(PairCtx c, bool active, uint32_t slot, uint32_t a, uint32_t b, bool cylinder_first, float query) {
    const uint32_t lane = c.lane, r = lane & 15u, gbase = lane & ~15u;
    const uint32_t cyl = cylinder_first ? a : b, plane = cylinder_first ? b : a;
    const BodyFrame fc = load_frame(c, cyl), fp = load_frame(c, plane);
    const float* sp = ctx_shape(c, cyl);
    const float radius = sp[0], half = sp[1];
    const V3 n = unit_or(fp.cz, mk3(0.f, 0.f, 1.f));
    const V3 axis = fc.cz;
    const float d = dot(axis, n);
    const bool on_cap = (d < 0.f ? -d : d) >= 0.95f;
    const V3 down = unit_or(axis * d - n, fc.cx);
    // lane -> (cap, rim step): the cap whose outward axis points against the plane normal carries the disk
    const int cap = on_cap ? (d > 0.f ? 1 : 0) : (int)(r & 1u);
    const int k = on_cap ? (int)r - 1 : -1;
    const bool exists = on_cap ? r < 9u : r < 2u;
    const float kS = 0.70710678f;
    const int kc = k & 7, ks = (k + 6) & 7;          // sin(k 45 deg) = cos((k - 2) 45 deg)
    auto octant_cos = [&](int i) { return i == 0 ? 1.0f : ((i == 1 || i == 7) ? kS : ((i == 2 || i == 6) ? 0.0f : ((i == 3 || i == 5) ? -kS : -1.0f))); };
    const V3 rim = fc.cx * octant_cos(kc) + fc.cy * octant_cos(ks);
    const V3 centre = fc.t + axis * (cap == 0 ? half : -half);
    const V3 p = centre + (k < 0 ? down : rim) * radius;
    const float sd = dot(p - fp.t, n);
    const bool touching = active && exists && sd < query;
    const float pen = -sd;
    const V3 pos = p - n * (sd * 0.5f);
    const uint32_t feature = k < 0 ? (uint32_t)cap : (uint32_t)(2 + cap * 8 + k);
    const uint32_t cand_mask = (__ballot_sync(NKB_FULL, touching) >> gbase) & 0xffffu;
    const uint32_t n_cand = __popc(cand_mask);
    uint32_t kept_mask = cand_mask;
    {
        float seed_pen = -3.4e38f;
        int seed = -1;
#pragma unroll
        for (int i = 0; i < 9; ++i) {
            const float pi = __shfl_sync(NKB_FULL, pen, gbase + i);
            if (((cand_mask >> i) & 1u) != 0u && (seed < 0 || pi > seed_pen)) { seed_pen = pi; seed = i; }
        }
        uint32_t spread = seed >= 0 ? 1u << seed : 0u;
        float nearest = 3.4e38f;
        int last = seed < 0 ? 0 : seed;
#pragma unroll 1
        for (int round = 1; round < 4; ++round) {
            const V3 K = mk3(__shfl_sync(NKB_FULL, pos.x, gbase + last), __shfl_sync(NKB_FULL, pos.y, gbase + last), __shfl_sync(NKB_FULL, pos.z, gbase + last));
            const V3 gap = pos - K;
            nearest = fminf(nearest, dot(gap, gap));
            float far = -1.0f;
            int pick = -1;
#pragma unroll
            for (int i = 0; i < 9; ++i) {
                const float mi = __shfl_sync(NKB_FULL, nearest, gbase + i);
                if (((cand_mask >> i) & 1u) != 0u && ((spread >> i) & 1u) == 0u && mi > far) { far = mi; pick = i; }
            }
            if (pick >= 0) { spread |= 1u << pick; last = pick; }
        }
        if (n_cand > 4u) kept_mask = spread;
    }
    if (touching && ((kept_mask >> r) & 1u) != 0u)
        write_point(c, slot, __popc(kept_mask & ((1u << r) - 1u)), a, b, pos, cylinder_first ? n : -n, pen, feature);
    if (active && r == 0u) ctx_count(c)[slot] = n_cand < 4u ? n_cand : 4u;
}

// ---- box on box: 16 lanes ----
static __device__ __noinline__ void box_box_group(PairCtx c, bool active, uint32_t slot, uint32_t a, uint32_t b, float query) {
    const uint32_t lane = c.lane, r = lane & 15u, gbase = lane & ~15u, group = lane >> 4;
    // frames are read from the shared-memory cache where they are needed (by run-time axis index) rather than held in registers
    const float* pa = ctx_shape(c, a);
    const float* pb = ctx_shape(c, b);
    const V3 ha = mk3(pa[0], pa[1], pa[2]), hb = mk3(pb[0], pb[1], pb[2]);
    const V3 between = frame_vec(c, b, 3) - frame_vec(c, a, 3);
    // --- lane r evaluates separating-axis candidate r: 0-2 faces of A, 3-5 faces of B, 6-14 edge crosses (A_i x B_j, i major) ---
    float pen = 0.f;
    V3 axis = mk3(0.f, 1.f, 0.f);
    bool usable = r < 15u;
    if (r < 6u) {
        const bool of_a = r < 3u;
        const int k = (int)(of_a ? r : r - 3u);
        const uint32_t own = of_a ? a : b, other = of_a ? b : a;
        const V3 u = frame_vec(c, own, k);
        // extent of the other box along u with the reference's |cos| + 1e-6 padding; the own box contributes its half extent
        const V3 oh = of_a ? hb : ha;
        const float c0 = fabsf(dot(u, frame_vec(c, other, 0))) + 1.0e-6f;
        const float c1 = fabsf(dot(u, frame_vec(c, other, 1))) + 1.0e-6f;
        const float c2 = fabsf(dot(u, frame_vec(c, other, 2))) + 1.0e-6f;
        const float reach_other = oh.x * c0 + oh.y * c1 + oh.z * c2;
        const float reach_own = comp(of_a ? ha : hb, k);
        const float d = dot(between, u);
        pen = (of_a ? reach_own + reach_other : reach_other + reach_own) - fabsf(d);
        axis = d < 0.f ? -u : u;
    } else if (r < 15u) {
        const int i = (int)(r - 6u) / 3, j = (int)(r - 6u) % 3;
        V3 u = cross(frame_vec(c, a, i), frame_vec(c, b, j));
        const float ll = len3(u);
        usable = ll >= 1.0e-6f;
        if (usable) {
            u = mk3(u.x / ll, u.y / ll, u.z / ll);
            const float ra = ha.x * fabsf(dot(frame_vec(c, a, 0), u)) + ha.y * fabsf(dot(frame_vec(c, a, 1), u)) + ha.z * fabsf(dot(frame_vec(c, a, 2), u));
            const float rb = hb.x * fabsf(dot(frame_vec(c, b, 0), u)) + hb.y * fabsf(dot(frame_vec(c, b, 1), u)) + hb.z * fabsf(dot(frame_vec(c, b, 2), u));
            const float d = dot(between, u);
            pen = (ra + rb) - fabsf(d);
            axis = d < 0.f ? -u : u;
        }
    }
    const uint32_t group_bits = 0xffffu << gbase;
    const bool apart = (__ballot_sync(NKB_FULL, usable && pen <= -query) & group_bits) != 0u;
    // --- the axis of least penetration, earlier candidates preferred unless a later one is better by more than 1e-5 ---
    float least = 3.4e38f;
    int best = -1;
#pragma unroll
    for (int k = 0; k < 15; ++k) {
        const float pk = __shfl_sync(NKB_FULL, pen, gbase + k);
        const bool uk = __shfl_sync(NKB_FULL, (int)usable, gbase + k) != 0;
        if (uk && pk < least - 1.0e-5f) { least = pk; best = k; }
    }
    const uint32_t best_lane = gbase + (uint32_t)(best < 0 ? 0 : best);
    const V3 normal_axis = mk3(__shfl_sync(NKB_FULL, axis.x, best_lane), __shfl_sync(NKB_FULL, axis.y, best_lane), __shfl_sync(NKB_FULL, axis.z, best_lane));
    const bool contact = active && !apart && best >= 0;
    const bool edge_case = best >= 6;
    // --- edge against edge: the closest points of the two supporting edges, one point ---
    if (contact && edge_case && r == 0u) {
        const int i = (best - 6) / 3, j = (best - 6) % 3;
        V3 on_a = frame_vec(c, a, 3), on_b = frame_vec(c, b, 3);
        for (int k = 0; k < 3; ++k) {
            const V3 ak = frame_vec(c, a, k);
            if (k != i) on_a = on_a + ak * ((dot(ak, normal_axis) >= 0.f ? 1.f : -1.f) * comp(ha, k));
        }
        for (int k = 0; k < 3; ++k) {
            const V3 bk = frame_vec(c, b, k);
            if (k != j) on_b = on_b + bk * ((dot(bk, normal_axis) >= 0.f ? -1.f : 1.f) * comp(hb, k));
        }
        const V3 da = frame_vec(c, a, i), db = frame_vec(c, b, j), gap = on_a - on_b;
        const float mix = dot(da, db), ga = dot(da, gap), gb = dot(db, gap), denom = 1.f * 1.f - mix * mix;
        float sa = 0.f, sb = 0.f;
        if (denom > 1.0e-9f) { sa = (mix * gb - 1.f * ga) / denom; sb = (1.f * gb - mix * ga) / denom; }
        const float ea = comp(ha, i), eb = comp(hb, j);
        sa = sa < -ea ? -ea : (sa > ea ? ea : sa);
        sb = sb < -eb ? -eb : (sb > eb ? eb : sb);
        write_point(c, slot, 0u, a, b, ((on_a + da * sa) + (on_b + db * sb)) * 0.5f, normal_axis, least, 0xE0000000u | ((uint32_t)i << 4) | (uint32_t)j);
        ctx_count(c)[slot] = 1u;
    }
    // --- face against face: the incident face (the other box's face most against the reference normal) clipped by the four side
    // --- planes of the reference face, lane v < 8 = polygon vertex v.  Runs for every group (shuffles need the whole warp); only
    // --- face contacts store anything. ---
    const bool ref_is_a = best < 3;
    const int ref_axis = best < 0 ? 0 : (ref_is_a ? best : (best < 6 ? best - 3 : 0));
    const uint32_t R = ref_is_a ? a : b, I = ref_is_a ? b : a;          // reference and incident box
    const V3 rh = ref_is_a ? ha : hb, ih = ref_is_a ? hb : ha;
    V3 ref_n = frame_vec(c, R, ref_axis);
    if (dot(frame_vec(c, I, 3) - frame_vec(c, R, 3), ref_n) < 0.f) ref_n = -ref_n;
    int inc_axis = 0;
    float most = 3.4e38f, inc_side = 1.f;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const float d = dot(frame_vec(c, I, k), ref_n), ad = fabsf(d);
        if (-ad < most) { most = -ad; inc_axis = k; inc_side = d < 0.f ? 1.f : -1.f; }
    }
    const int iu = (inc_axis + 1) % 3, iv = (inc_axis + 2) % 3;
    const V3 inc_centre = frame_vec(c, I, 3) + frame_vec(c, I, inc_axis) * (inc_side * comp(ih, inc_axis));
    const uint32_t v = r & 7u;
    // quad corners in the order (-,-) (+,-) (+,+) (-,+) of the incident face's own axes
    const float su = (v == 1u || v == 2u) ? 1.f : -1.f, sv = (v >= 2u) ? 1.f : -1.f;
    V3 P = inc_centre + frame_vec(c, I, iu) * (su * comp(ih, iu)) + frame_vec(c, I, iv) * (sv * comp(ih, iv));
    uint32_t count = 4u;
    const int ru = (ref_axis + 1) % 3, rv = (ref_axis + 2) % 3;
    const float eu = comp(rh, ru), ev = comp(rh, rv);
    const V3 ref_centre = frame_vec(c, R, 3) + ref_n * comp(rh, ref_axis);
    float* stage = ctx_clip_stage(c, group);
    const uint32_t vbase = gbase;                  // polygon lanes are the group's first eight
#pragma unroll 1
    for (int side = 0; side < 4; ++side) {
        const V3 along = frame_vec(c, R, side < 2 ? ru : rv);
        const float extent = side < 2 ? eu : ev;
        const V3 pn = (side & 1) == 0 ? along : -along;
        const V3 pp = (side & 1) == 0 ? ref_centre + along * extent : ref_centre - along * extent;
        const float dc = dot(P - pp, pn);
        const uint32_t next = count != 0u ? (v + 1u) % count : 0u;
        const V3 Q = mk3(__shfl_sync(NKB_FULL, P.x, vbase + next), __shfl_sync(NKB_FULL, P.y, vbase + next), __shfl_sync(NKB_FULL, P.z, vbase + next));
        const float dn = __shfl_sync(NKB_FULL, dc, vbase + next);
        const bool live = r < 8u && v < count;
        const bool in_c = dc <= 0.f, in_n = dn <= 0.f;
        const uint32_t keep = live && in_c ? 1u : 0u, cut = live && (in_c != in_n) ? 1u : 0u;
        uint32_t upto = keep + cut;                 // inclusive prefix over the eight polygon lanes
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) { const uint32_t up = __shfl_up_sync(NKB_FULL, upto, o, 8); if ((int)v >= o) upto += up; }
        const uint32_t first = upto - (keep + cut);
        const uint32_t total = __shfl_sync(NKB_FULL, upto, vbase + 7u);
        if (keep != 0u && first < 8u) st3(stage + 4u * first, P);
        if (cut != 0u && first + keep < 8u) {
            const float tt = dc / (dc - dn);
            st3(stage + 4u * (first + keep), mk3(P.x + (Q.x - P.x) * tt, P.y + (Q.y - P.y) * tt, P.z + (Q.z - P.z) * tt));
        }
        __syncwarp();
        count = total < 8u ? total : 8u;
        if (r < 8u && v < count) P = ld3(stage + 4u * v);
        __syncwarp();
    }
    const float depth = dot(ref_centre - P, ref_n);
    const bool candidate = contact && !edge_case && r < 8u && v < count && depth >= -query;
    const uint32_t cand_mask = (__ballot_sync(NKB_FULL, candidate) >> vbase) & 0xffu;
    const uint32_t n_cand = __popc(cand_mask);
    const V3 mid = (P + (P + ref_n * depth)) * 0.5f;
    const V3 out_normal = ref_is_a ? -ref_n : ref_n;
    // farthest-point spread when more than four candidates: the deepest (lowest index on ties) seeds, then three times the
    // candidate farthest from everything kept so far (lowest index on ties)
    uint32_t kept_mask = cand_mask;
    {
        float seed_pen = -3.4e38f;
        int seed = -1;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float pk = __shfl_sync(NKB_FULL, depth, vbase + k);
            if (((cand_mask >> k) & 1u) != 0u && (seed < 0 || pk > seed_pen)) { seed_pen = pk; seed = k; }
        }
        uint32_t spread = seed >= 0 ? 1u << seed : 0u;
        float nearest = 3.4e38f;                    // this lane's squared distance to the kept set
        int last = seed < 0 ? 0 : seed;
#pragma unroll 1
        for (int round = 1; round < 4; ++round) {
            const V3 K = mk3(__shfl_sync(NKB_FULL, mid.x, vbase + last), __shfl_sync(NKB_FULL, mid.y, vbase + last), __shfl_sync(NKB_FULL, mid.z, vbase + last));
            const V3 d = mid - K;
            nearest = fminf(nearest, dot(d, d));
            float far = -1.0f;
            int pick = -1;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float mk = __shfl_sync(NKB_FULL, nearest, vbase + k);
                if (((cand_mask >> k) & 1u) != 0u && ((spread >> k) & 1u) == 0u && mk > far) { far = mk; pick = k; }
            }
            if (pick >= 0) { spread |= 1u << pick; last = pick; }
        }
        if (n_cand > 4u) kept_mask = spread;
    }
    if (candidate && ((kept_mask >> v) & 1u) != 0u)
        write_point(c, slot, __popc(kept_mask & ((1u << v) - 1u)), a, b, mid, out_normal, depth, v);
    if (contact && !edge_case && r == 0u) {
        if (n_cand == 0u) {         // the clipped face lies beyond the query band everywhere: one point under the incident face centre
            write_point(c, slot, 0u, a, b, inc_centre + ref_n * (least * 0.5f), out_normal, least, (uint32_t)inc_axis << 4);
            ctx_count(c)[slot] = 1u;
        } else ctx_count(c)[slot] = n_cand < 4u ? n_cand : 4u;
    }
    if (active && !contact && r == 0u) ctx_count(c)[slot] = 0u;
}

// One world frame per collidable row, cached in the narrowphase scratch for every pair that touches the body.
NKB_DEV void narrowphase_frames(Env& e) {
    const TemplateView& t = *e.t;
    const PairCtx c = pair_ctx(e, 0.f);
    for (uint32_t b = e.lane; b < t.B; b += 32u) {
        const float* bp = sm_bpose(e, b);
        const Q4 q = ldq(bp + 3);
        float* f = ctx_frames(c) + 12u * b;
        st3(f, qrot_raw(q, mk3(1.f, 0.f, 0.f))); st3(f + 3, qrot_raw(q, mk3(0.f, 1.f, 0.f))); st3(f + 6, qrot_raw(q, mk3(0.f, 0.f, 1.f)));
        st3(f + 9, ld3(bp));
    }
    __syncwarp();
}

// Contact manifolds of the candidate slots: points, normals, depths (+ the separation shell), identities, counts.
// Range form: this warp takes the 32-slot batches first, first + stride, ... (the frames are cached beforehand).
NKB_DEV void narrowphase_range(Env& e, uint32_t pair_count, uint32_t first, uint32_t stride) {
    const TemplateView& t = *e.t;
    const float separation = fmaxf(t.cfg.contact_margin, 0.0005f), reach = query_reach(t.cfg);
    const uint32_t S = t.slot_cap, lane = e.lane;          // slots past the admissible-pair count can never fill and have no storage
    PairCtx c = pair_ctx(e, separation);
    c.stage_shift = 64u * first;
    for (uint32_t base = 32u * first; base < S; base += 32u * stride) {
        const uint32_t s = base + lane;
        const bool live = s < pair_count;
        uint32_t a = 0u, b = 0u, ka = kSphere, kb = kSphere, cls = kClassNone;
        float query = 0.f;
        if (live) {
            const uint32_t ab = sm_pairs(e)[s];
            a = ab >> 16; b = ab & 0xffffu;
            ka = __ldg(t.shape_kind + a); kb = __ldg(t.shape_kind + b);
            cls = pair_class(ka, kb);
            query = fmaxf(separation, fminf(motion_radius(2.0f * separation, t.cfg.dt, body_speed(e, a), body_speed(e, b)), reach));
        }
        if (s < S && cls != kClassBoxPlane && cls != kClassBoxBox && cls != kClassCylinderPlane) {
            uint32_t count = 0u;
            if (cls == kClassRound) {
                RoundPoints pts;
                round_pair(ka, load_frame(c, a), t.shape_params + 4u * a, kb, load_frame(c, b), t.shape_params + 4u * b, query, pts);
                count = pts.count;
                if (count > 0u) write_point(c, s, 0u, a, b, pts.pos[0], pts.normal, pts.pen[0], pts.key[0]);
                if (count > 1u) write_point(c, s, 1u, a, b, pts.pos[1], pts.normal, pts.pen[1], pts.key[1]);
            }
            ctx_count(c)[s] = count;
        }
        // box on plane: four pairs per pass, eight lanes each
        for (uint32_t todo = __ballot_sync(NKB_FULL, cls == kClassBoxPlane); todo != 0u;) {
            const uint32_t owner = nth_set_bit(todo, lane >> 3);
            const bool active = owner < 32u;
            const uint32_t src = active ? owner : 0u;
            const uint32_t ga = __shfl_sync(NKB_FULL, a, src), gb = __shfl_sync(NKB_FULL, b, src), gka = __shfl_sync(NKB_FULL, ka, src);
            const float gq = __shfl_sync(NKB_FULL, query, src);
            box_plane_group(c, active, base + src, ga, gb, gka == kBox, gq);
            for (int k = 0; k < 4 && todo != 0u; ++k) todo &= todo - 1u;
        }
        // cylinder on plane: two pairs per pass, sixteen lanes each
        for (uint32_t todo = __ballot_sync(NKB_FULL, cls == kClassCylinderPlane); todo != 0u;) {
            const uint32_t owner = nth_set_bit(todo, lane >> 4);
            const bool active = owner < 32u;
            const uint32_t src = active ? owner : 0u;
            const uint32_t ga = __shfl_sync(NKB_FULL, a, src), gb = __shfl_sync(NKB_FULL, b, src), gka = __shfl_sync(NKB_FULL, ka, src);
            const float gq = __shfl_sync(NKB_FULL, query, src);
            cylinder_plane_group(c, active, base + src, ga, gb, gka == kCylinder, gq);
            for (int k = 0; k < 2 && todo != 0u; ++k) todo &= todo - 1u;
        }
        // box on box: two pairs per pass, sixteen lanes each
        for (uint32_t todo = __ballot_sync(NKB_FULL, cls == kClassBoxBox); todo != 0u;) {
            const uint32_t owner = nth_set_bit(todo, lane >> 4);
            const bool active = owner < 32u;
            const uint32_t src = active ? owner : 0u;
            const uint32_t ga = __shfl_sync(NKB_FULL, a, src), gb = __shfl_sync(NKB_FULL, b, src);
            const float gq = __shfl_sync(NKB_FULL, query, src);
            box_box_group(c, active, base + src, ga, gb, gq);
            for (int k = 0; k < 2 && todo != 0u; ++k) todo &= todo - 1u;
        }
    }
    __syncwarp();
}

}  // namespace nkb
