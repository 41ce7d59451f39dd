// Warp-per-env constraint heads: contact rows (normal + two tangents per point), joint limit, joint friction and
// drive rows, chain Jacobians of articulated sides, and the contact warm-start cache.
// A "head" is one solver row group; its state lives in shared memory as a structure of arrays so that one
// lane can own one head.  Quantities follow the reference's ops/assemble_rows.cu:406-801 (contact rows),
// :805-971 (joint rows), :122-186 (chain Jacobians), ops/articulation_types.cuh:193-238 and the warm-start
// behaviour of ops/assemble_rows.cu:1228-1391 with ops/contact_cache.cuh.
#pragma once
#include "nkb_collide.cuh"

namespace nkb {

// head fields (word offsets inside a head record)
enum HeadField : uint32_t {
    HF_FLAGS = 0, HF_OWNER, HF_REF, HF_JOFF, HF_UNITV,
    HF_RHO, HF_RSD, HF_RSR, HF_LOWER, HF_UPPER, HF_MU, HF_NB, HF_PEN, HF_RHS,
    HF_DUAL, HF_BASE = HF_DUAL + 3, HF_RES = HF_BASE + 3, HF_MOVE = HF_RES + 3, HF_STEP = HF_MOVE + 3,
    HF_RXS = HF_STEP + 3, HF_RXW = HF_RXS + 3, HF_RXP,
    HF_N = HF_RXP + 3, HF_T1 = HF_N + 3, HF_T2 = HF_T1 + 3, HF_RA = HF_T2 + 3, HF_RB = HF_RA + 3,
    HF_LAM = HF_RB + 3,          // physical multipliers after the velocity solve
    HF_F = HF_LAM + 3,           // response impulse, curvature (xx, yy, zz, yz) and noise scale at the current move
    HF_C = HF_F + 3, HF_NZ = HF_C + 4,
    HF_COUNT = HF_NZ + 3
};
constexpr uint32_t kNoBlock16 = 0xffffu;
constexpr uint32_t kUnitRow = 0x80000000u;   // HF_JOFF: unit row on coordinate (value & 0xffff)

// heads are records of kHeadStride words (odd, so one lane per head is conflict-free and fields are immediate offsets)
NKB_DEV float& hf(const Env& e, uint32_t field, uint32_t h) { return e.sm[e.lay->heads + h * kHeadStride + field]; }
NKB_DEV uint32_t& hu(const Env& e, uint32_t field, uint32_t h) { return reinterpret_cast<uint32_t*>(e.sm)[e.lay->heads + h * kHeadStride + field]; }
NKB_DEV V3 hf3(const Env& e, uint32_t field, uint32_t h) { return mk3(hf(e, field, h), hf(e, field + 1u, h), hf(e, field + 2u, h)); }
NKB_DEV void hst3(const Env& e, uint32_t field, uint32_t h, V3 v) { hf(e, field, h) = v.x; hf(e, field + 1u, h) = v.y; hf(e, field + 2u, h) = v.z; }
NKB_DEV float* sm_jpool(const Env& e) { return e.sm + e.lay->jpool; }

NKB_DEV void tangent_basis(V3 normal, V3& t1, V3& t2) {
    const float ls = dot(normal, normal);
    const V3 n = ls > 1.0e-10f ? normal * rsqrtf(ls) : mk3(0.f, 0.f, 1.f);
    V3 ref = mk3(1.f, 0.f, 0.f);
    if (fabsf(n.x) > 0.9f) ref = mk3(0.f, 1.f, 0.f);
    const float proj = dot(ref, n);
    V3 ta = mk3(ref.x - proj * n.x, ref.y - proj * n.y, ref.z - proj * n.z);
    const float l2 = dot(ta, ta);
    if (l2 > 1.0e-12f) ta = ta * rsqrtf(l2); else ta = mk3(1.f, 0.f, 0.f);
    t1 = ta; t2 = cross(n, ta);
}

// Block index of a collidable row's owner: free body -> its row, link mirror -> B (the articulation), else none.
NKB_DEV uint32_t side_block(const Env& e, uint32_t body, uint32_t& link) {
    const TemplateView& t = *e.t;
    link = kNoLink;
    if (__ldg(t.body_id + body) < 0) return kNoBlock16;
    const uint32_t l = __ldg(t.body_to_link + body);
    if (l == kNoLink) return __ldg(t.inv_mass + body) > 0.f ? body : kNoBlock16;
    link = l;
    return t.ndof != 0u ? t.B : kNoBlock16;
}

// Builds every head of the env.  Returns the head count (capped at head_cap).
template <int NR>
NKB_DEV uint32_t stage_rows(Env& e, uint32_t pair_count) {
    const TemplateView& t = *e.t;
    const uint32_t S = t.cfg.max_contacts, n = t.ndof, L = t.L, lane = e.lane;
    const float dt = t.cfg.dt;
    const bool position_pass = t.cfg.pos_iters > 0u;
    uint32_t nheads = 0u, npoints = 0u;
    // contact heads in slot order
    for (uint32_t base = 0u; base < S; base += 32u) {
        const uint32_t s = base + lane;
        const uint32_t cnt = (s < S && s < pair_count) ? sm_ccount(e)[s] : 0u;
        uint32_t incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(NKB_FULL, incl, o); if ((int)lane >= o) incl += v; }
        const uint32_t first = nheads + incl - cnt;
        const uint32_t total = __shfl_sync(NKB_FULL, incl, 31);
        if (cnt != 0u) {
            const uint32_t ab = sm_pairs(e)[s], a = ab >> 16, b = ab & 0xffffu;
            uint32_t la, lb;
            const uint32_t oa = side_block(e, a, la), ob = side_block(e, b, lb);
            V3 com_a = mk3(0.f, 0.f, 0.f), com_b = com_a;
            if (oa < t.B) com_a = ld3(sm_bpose(e, a)) + qrot(ldq(sm_bpose(e, a) + 3), ld3(t.inertial_pos + 3u * a));
            if (ob < t.B) com_b = ld3(sm_bpose(e, b)) + qrot(ldq(sm_bpose(e, b) + 3), ld3(t.inertial_pos + 3u * b));
            const float mu = fmaxf(__ldg(t.mu + a), __ldg(t.mu + b));
            for (uint32_t p = 0u; p < cnt; ++p) {
                const uint32_t h = first + p, at = s * 4u + p;
                if (h >= t.head_cap || h >= t.point_cap) { e.status |= kStatusHeadOverflow; continue; }
                const V3 raw = ld3(sm_cnormal(e, at)), point = ld3(sm_cpoint(e, at));
                const float len = sqrtf(raw.x * raw.x + raw.y * raw.y + raw.z * raw.z);
                const V3 nn = len < 1e-12f ? mk3(0.f, 0.f, 0.f) : mk3(raw.x / len, raw.y / len, raw.z / len);
                V3 t1, t2; tangent_basis(raw, t1, t2);
                const float cd = sm_cdepth(e)[at];
                const V3 ext = mk3(fabsf(point.x) + fabsf(nn.x * cd), fabsf(point.y) + fabsf(nn.y * cd), fabsf(point.z) + fabsf(nn.z * cd));
                const double gamma = 3.0 * (double)FLT_EPSILON / (1.0 - 3.0 * (double)FLT_EPSILON);
                const double roundoff = gamma * (fabs((double)nn.x) * (2.0 * fabs((double)ext.x)) + fabs((double)nn.y) * (2.0 * fabs((double)ext.y)) +
                                                 fabs((double)nn.z) * (2.0 * fabs((double)ext.z)));
                const float clearance = roundoff > 0.0 ? __int_as_float(__float_as_int((float)roundoff) + 1) : 0.0f;     // next float up
                const float depth = cd + clearance;
                hu(e, HF_FLAGS, h) = kHeadContact | kHeadContactNormal | kHeadSpeculative;
                const uint32_t own1 = ob == oa ? kNoBlock16 : ob;
                hu(e, HF_OWNER, h) = oa | (own1 << 16);
                hu(e, HF_REF, h) = at | (la != kNoLink ? (la << 16) : 0xffff0000u);
                hu(e, HF_JOFF, h) = lb != kNoLink ? lb : 0xffffu;      // side-b link, pool offset is filled below
                hf(e, HF_UNITV, h) = 0.f;
                hf(e, HF_LOWER, h) = 0.f; hf(e, HF_UPPER, h) = FLT_MAX; hf(e, HF_MU, h) = mu;
                hf(e, HF_PEN, h) = depth;
                hf(e, HF_RHS, h) = (fminf(depth, 0.0f) + (position_pass ? 0.0f : fminf(fmaxf(cd, 0.0f), t.cfg.overlap_recovery_velocity * dt))) / (dt * dt);
                hst3(e, HF_N, h, nn); hst3(e, HF_T1, h, t1); hst3(e, HF_T2, h, t2);
                hst3(e, HF_RA, h, point - com_a); hst3(e, HF_RB, h, point - com_b);
                hst3(e, HF_DUAL, h, mk3(0.f, 0.f, 0.f));
            }
        }
        nheads += total;
        npoints += total;
    }
    if (nheads > t.head_cap) nheads = t.head_cap;
    if (nheads > t.point_cap) nheads = t.point_cap;
    const uint32_t ncontact = nheads;
    __syncwarp();
    // chain Jacobians of articulated sides, lane = coordinate (ops/articulation_types.cuh:193-238)
    if (n != 0u && ncontact != 0u) {
        V3 axis_w[NR], origin[NR];
        uint32_t jt[NR];
        bool dof[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            axis_w[r] = mk3(0.f, 0.f, 0.f); origin[r] = axis_w[r];
            jt[r] = kFixed;
            dof[r] = lane + 32u * r < n;
            if (dof[r]) {
                const uint32_t dl = e.dof_link[r];
                jt[r] = __ldg(t.jtype + dl);
                if (jt[r] == kFloating) {
                    const float* bp = e.s->base_pose + (size_t)e.env * 7u;
                    const Q4 br = ldq(bp + 3);
                    const uint32_t c = e.dof_comp[r] % 3u;
                    axis_w[r] = qrot(br, mk3(c == 0u ? 1.f : 0.f, c == 1u ? 1.f : 0.f, c == 2u ? 1.f : 0.f));
                    origin[r] = ld3(bp);
                } else {
                    V3 a = ld3(t.axis + 3u * dl);
                    axis_w[r] = qrot(ldq(sm_pose(e, dl) + 3), a);
                    origin[r] = ld3(sm_pose(e, dl));
                }
            }
        }
        float* pool = sm_jpool(e);
        for (uint32_t h = 0u; h < ncontact; ++h) {
            const uint32_t ref = hu(e, HF_REF, h), la = ref >> 16, lb = hu(e, HF_JOFF, h) & 0xffffu;
            __syncwarp();      // every lane has read the side-b link before lane 0 replaces it with the pool offset
            const uint32_t n4 = (n + 3u) & ~3u, joff = h * 3u * n4;
            const V3 point = ld3(sm_cpoint(e, ref & 0xffffu));
            const V3 dirs[3] = {hf3(e, HF_N, h), hf3(e, HF_T1, h), hf3(e, HF_T2, h)};
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t c = lane + 32u * r;
                if (dof[r]) {
                    float ent[3] = {0.f, 0.f, 0.f};
#pragma unroll
                    for (int side = 0; side < 2; ++side) {
                        const uint32_t cl = side == 0 ? la : lb;
                        if (cl == 0xffffu) continue;
                        if (!((__ldg(t.anc_mask + cl) >> e.dof_link[r]) & 1u)) continue;
                        const float sgn = side == 0 ? 1.f : -1.f;
#pragma unroll
                        for (int ax = 0; ax < 3; ++ax) {
                            const V3 f = dirs[ax] * sgn;
                            float v;
                            if (jt[r] == kFloating) v = e.dof_comp[r] < 3u ? dot(cross(axis_w[r], point - origin[r]), f) + 0.0f : dot(axis_w[r], f);
                            else if (jt[r] == kPrismatic) v = dot(axis_w[r], f);
                            else v = dot(cross(axis_w[r], point - origin[r]), f) + 0.0f;
                            ent[ax] += v;
                        }
                    }
                    pool[joff + c] = ent[0]; pool[joff + n4 + c] = ent[1]; pool[joff + 2u * n4 + c] = ent[2];
                } else if (c < n4) { pool[joff + c] = 0.f; pool[joff + n4 + c] = 0.f; pool[joff + 2u * n4 + c] = 0.f; }
            }
            if (lane == 0u) hu(e, HF_JOFF, h) = joff;
        }
    }
    __syncwarp();
    // joint rows, lane = link: limit lower/upper, dry friction, drive (ops/assemble_rows.cu:805-971)
    for (uint32_t kind = 0u; kind < 4u; ++kind) {
        bool emit = false;
        float lower = 0.f, upper = 0.f, rhs = 0.f, pen = 0.f, unitv = 1.f, lambda = 0.f;
        uint32_t flags = 0u;
        if (lane < L && joint_dofs(e.jtype) == 1u) {
            const uint32_t lf = __ldg(t.limit_flags + lane);
            if (kind < 2u && (lf & (1u << kind))) {
                const float bound = kind == 0u ? __ldg(t.limit_lower + lane) : __ldg(t.limit_upper + lane);
                const float dist = kind == 0u ? e.q - bound : bound - e.q;
                const float target = -(position_pass ? fmaxf(dist, 0.0f) : dist) / dt;
                emit = true; flags = kHeadLimit; unitv = kind == 0u ? 1.f : -1.f;
                rhs = fminf(target, t.cfg.baumgarte_max_velocity) / dt;
                lower = 0.f; upper = FLT_MAX; pen = fmaxf(-dist, 0.0f);
            } else if (kind == 2u) {
                const float fr = __ldg(t.frictionloss + lane);
                if (fr > 0.f) { emit = true; flags = kHeadFriction | kHeadVelocityOnly; lower = -fr * dt; upper = fr * dt; }
            } else if (kind == 3u) {
                const float effort = fminf(fmaxf(e.drive_command, e.drive_lower), e.drive_upper);
                if (effort != 0.f) { emit = true; flags = kHeadDrive | kHeadVelocityOnly; lower = upper = effort * dt; lambda = lower; }
            }
        }
        // limit rows interleave lower/upper per link: kinds 0 and 1 are placed together
        if (kind == 0u) {
            // count both limit kinds per link so that a link's lower row precedes its upper row
            const uint32_t lf = (lane < L && joint_dofs(e.jtype) == 1u) ? (__ldg(t.limit_flags + lane) & 3u) : 0u;
            const uint32_t cnt = __popc(lf);
            uint32_t incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(NKB_FULL, incl, o); if ((int)lane >= o) incl += v; }
            const uint32_t first = nheads + incl - cnt;
            const uint32_t total = __shfl_sync(NKB_FULL, incl, 31);
            for (uint32_t side = 0u; side < 2u; ++side) {
                if (!(lf & (1u << side))) continue;
                const uint32_t h = first + ((side == 1u && (lf & 1u)) ? 1u : 0u);
                if (h >= t.head_cap) { e.status |= kStatusHeadOverflow; continue; }
                const float bound = side == 0u ? __ldg(t.limit_lower + lane) : __ldg(t.limit_upper + lane);
                const float dist = side == 0u ? e.q - bound : bound - e.q;
                const float target = -(position_pass ? fmaxf(dist, 0.0f) : dist) / dt;
                hu(e, HF_FLAGS, h) = kHeadLimit;
                hu(e, HF_OWNER, h) = t.B | (kNoBlock16 << 16);
                hu(e, HF_REF, h) = lane;
                hu(e, HF_JOFF, h) = kUnitRow | e.link_dof;
                hf(e, HF_UNITV, h) = side == 0u ? 1.f : -1.f;
                hf(e, HF_LOWER, h) = 0.f; hf(e, HF_UPPER, h) = FLT_MAX; hf(e, HF_MU, h) = 0.f;
                hf(e, HF_PEN, h) = fmaxf(-dist, 0.0f);
                hf(e, HF_RHS, h) = fminf(target, t.cfg.baumgarte_max_velocity) / dt;
                // an authored limit row starts from the multiplier the last step's solve left in its slot: the reference
                // clears lambda only for links without that limit (ops/assemble_rows.cu:826-879; the per-step clear
                // :366-383 covers the contact rows alone)
                const float carried = e.s->limit_lambda[((size_t)e.env * L + lane) * 2u + side];
                hst3(e, HF_DUAL, h, mk3(carried, 0.f, 0.f));
                hst3(e, HF_LAM, h, mk3(carried, 0.f, 0.f));
            }
            nheads = min(nheads + total, t.head_cap);
            ++kind;       // kind 1 handled here
            continue;
        }
        const uint32_t mask = __ballot_sync(NKB_FULL, emit);
        const uint32_t h = nheads + __popc(mask & ((1u << lane) - 1u));
        if (emit) {
            if (h >= t.head_cap) e.status |= kStatusHeadOverflow;
            else {
                hu(e, HF_FLAGS, h) = flags;
                hu(e, HF_OWNER, h) = t.B | (kNoBlock16 << 16);
                hu(e, HF_REF, h) = lane;
                hu(e, HF_JOFF, h) = kUnitRow | e.link_dof;
                hf(e, HF_UNITV, h) = unitv;
                hf(e, HF_LOWER, h) = lower; hf(e, HF_UPPER, h) = upper; hf(e, HF_MU, h) = 0.f;
                hf(e, HF_PEN, h) = pen; hf(e, HF_RHS, h) = rhs;
                hst3(e, HF_DUAL, h, mk3(lambda, 0.f, 0.f));
            }
        }
        nheads = min(nheads + __popc(mask), t.head_cap);
    }
    __syncwarp();
    return nheads;
}

NKB_DEV uint32_t head_pair(const Env& e, uint32_t h) { return sm_pairs(e)[(hu(e, HF_REF, h) & 0xffffu) >> 2]; }

// Warm start (phase 0): a contact head takes the multipliers of the cached point with the same identity.
// Range form: this warp takes the heads first, first + stride, ... (a head's match reads earlier heads and the cache and
// writes only the head's own dual).
NKB_DEV void warm_start_range(Env& e, uint32_t nheads, uint32_t first, uint32_t stride) {
    const TemplateView& t = *e.t;
    const uint32_t npts = t.cfg.max_contacts * 4u;
    const CacheEntry* cache = e.s->cache + (size_t)e.env * npts;
    for (uint32_t h = first; h < nheads; h += stride) {
        if (!(hu(e, HF_FLAGS, h) & kHeadContact)) break;     // contact heads come first
        const uint32_t at = hu(e, HF_REF, h) & 0xffffu;
        const uint32_t pair = head_pair(e, h);
        const uint32_t* f = sm_cfeat(e, at);
        const unsigned long long feat = (unsigned long long)f[0] | ((unsigned long long)f[1] << 32);
        // an earlier current point with the same identity owns the match
        bool dup = false;
        for (uint32_t base = 0u; base < h; base += 32u) {
            const uint32_t j = base + e.lane;
            bool same = false;
            if (j < h) {
                const uint32_t* g = sm_cfeat(e, hu(e, HF_REF, j) & 0xffffu);
                same = head_pair(e, j) == pair && g[0] == f[0] && g[1] == f[1];
            }
            dup |= __any_sync(NKB_FULL, same);
        }
        if (dup) continue;
        uint32_t found = 0xffffffffu;
        for (uint32_t base = 0u; base < npts && found == 0xffffffffu; base += 32u) {
            const uint32_t c = base + e.lane;
            const bool hit = c < npts && cache[c].pair == pair && cache[c].feature == feat && cache[c].age < 2u;
            const uint32_t m = __ballot_sync(NKB_FULL, hit);
            if (m != 0u) found = base + (uint32_t)__ffs(m) - 1u;
        }
        if (found == 0xffffffffu) continue;
        if (e.lane == 0u) {
            const CacheEntry en = cache[found];
            const V3 nrm = ld3(sm_cnormal(e, at)), cn = mk3(en.normal[0], en.normal[1], en.normal[2]);
            if (dot(nrm, cn) > 0.25f) {
                V3 ot1, ot2, t1, t2;
                tangent_basis(cn, ot1, ot2);
                tangent_basis(nrm, t1, t2);
                const V3 old = ot1 * en.lambda[1] + ot2 * en.lambda[2];
                hst3(e, HF_DUAL, h, mk3(fmaxf(en.lambda[0], 0.0f), dot(old, t1), dot(old, t2)));
            }
        }
    }
    __syncwarp();
}

// Owner marks of the cache rebuild: the first current point of each identity owns its cache entry.  Range form over the
// contact heads first, first + stride, ... (a head's test reads earlier heads and writes its own point's mark).
NKB_DEV void cache_owners_range(Env& e, uint32_t ncontact, uint32_t first, uint32_t stride) {
    const TemplateView& t = *e.t;
    const uint32_t stage_cap = min(t.point_cap, t.slot_cap * 4u);
    uint32_t* owner = reinterpret_cast<uint32_t*>(reinterpret_cast<CacheEntry*>(e.sm + e.lay->cstage) + stage_cap);
    for (uint32_t h = first; h < ncontact; h += stride) {
        const uint32_t at = hu(e, HF_REF, h) & 0xffffu;
        const uint32_t pair = head_pair(e, h);
        const uint32_t* f = sm_cfeat(e, at);
        bool dup = false;
        for (uint32_t base = 0u; base < h; base += 32u) {
            const uint32_t j = base + e.lane;
            bool same = false;
            if (j < h) { const uint32_t* g = sm_cfeat(e, hu(e, HF_REF, j) & 0xffffu); same = head_pair(e, j) == pair && g[0] == f[0] && g[1] == f[1]; }
            dup |= __any_sync(NKB_FULL, same);
        }
        if (!dup && e.lane == 0u) owner[at] = h;
    }
    __syncwarp();
}

// Warm start (phase 1): rebuilds the env's cache from the solved multipliers; unmatched cached points of age 0
// survive one more step in the points no current contact owns.
template <typename Owners>
NKB_DEV void stage_cache_commit(Env& e, uint32_t nheads, Owners&& owners) {
    const TemplateView& t = *e.t;
    const uint32_t npts = t.cfg.max_contacts * 4u;
    if (npts == 0u) return;
    CacheEntry* cache = e.s->cache + (size_t)e.env * npts;
    CacheEntry* stage = reinterpret_cast<CacheEntry*>(e.sm + e.lay->cstage);
    // only points of fillable slots can own an entry, and a step retains at most the previous step's owners
    const uint32_t nown = t.slot_cap * 4u;
    const uint32_t stage_cap = min(t.point_cap, nown);
    uint32_t* owner = reinterpret_cast<uint32_t*>(stage + stage_cap);
    for (uint32_t c = e.lane; c < nown; c += 32u) owner[c] = 0xffffffffu;
    __syncwarp();
    // owners: first current point of each identity
    uint32_t ncontact = 0u;
    for (uint32_t base = 0u; base < nheads; base += 32u) {          // contact heads come first
        const uint32_t h = base + e.lane;
        const uint32_t m = __ballot_sync(NKB_FULL, h < nheads && (hu(e, HF_FLAGS, h) & kHeadContact) != 0u);
        ncontact += __popc(m);
        if (m != 0xffffffffu) break;
    }
    owners(ncontact);
    __syncwarp();
    // retained old entries in ascending cache order
    uint32_t nret = 0u;
    for (uint32_t base = 0u; base < npts; base += 32u) {
        const uint32_t c = base + e.lane;
        bool keep = false;
        CacheEntry en;
        en.pair = 0xffffffffu; en.feature = 0ull; en.age = 0u;
        if (c < npts) {
            en = cache[c];
            keep = en.pair != 0xffffffffu && en.age < 1u;
            for (uint32_t h = 0u; h < ncontact && keep; ++h) {
                const uint32_t* f = sm_cfeat(e, hu(e, HF_REF, h) & 0xffffu);
                if (head_pair(e, h) == en.pair && (((unsigned long long)f[1] << 32) | f[0]) == en.feature) keep = false;
            }
            for (uint32_t d = 0u; d < c && keep; ++d) if (cache[d].pair == en.pair && cache[d].feature == en.feature) keep = false;
        }
        const uint32_t m = __ballot_sync(NKB_FULL, keep);
        const uint32_t to = nret + __popc(m & ((1u << e.lane) - 1u));
        if (keep && to < stage_cap) { en.age += 1u; stage[to] = en; }
        nret = min(nret + __popc(m), stage_cap);
    }
    __syncwarp();
    // write the new cache: owners at their own point, retained entries into the free points in order
    uint32_t free_seen = 0u;
    for (uint32_t base = 0u; base < npts; base += 32u) {
        const uint32_t c = base + e.lane;
        const bool is_free = c < npts && (c >= nown || owner[c] == 0xffffffffu);
        const uint32_t m = __ballot_sync(NKB_FULL, is_free);
        if (c < npts) {
            CacheEntry en;
            if (!is_free) {
                const uint32_t h = owner[c];
                const uint32_t* f = sm_cfeat(e, c);
                en.pair = head_pair(e, h); en.feature = ((unsigned long long)f[1] << 32) | f[0]; en.age = 0u;
                const V3 lam = hf3(e, HF_LAM, h);
                en.lambda[0] = lam.x; en.lambda[1] = lam.y; en.lambda[2] = lam.z;
                const V3 nn = ld3(sm_cnormal(e, c));
                en.normal[0] = nn.x; en.normal[1] = nn.y; en.normal[2] = nn.z;
            } else {
                const uint32_t k = free_seen + __popc(m & ((1u << e.lane) - 1u));
                if (k < nret) en = stage[k];
                else { en.pair = 0xffffffffu; en.feature = 0ull; en.age = 0u; en.lambda[0] = en.lambda[1] = en.lambda[2] = 0.f; en.normal[0] = en.normal[1] = en.normal[2] = 0.f; }
            }
            cache[c] = en;
        }
        free_seen += __popc(m);
    }
    __syncwarp();
}

}  // namespace nkb
