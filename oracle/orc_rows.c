/* Oracle (test infrastructure): constraint row assembly and contact warm start.
 * Restates the reference's ops/assemble_rows.cu (EmitPairDrivenRowsKernel, EmitJointRowsKernel,
 * ComputeContactChainJacobianKernel, MergeSharedArticulationJacobianKernel), articulation_types.cuh
 * AccumulateChainJointForce and the functional behaviour of ops/contact_cache.cuh. */
#include "orc.h"
#include "orc_math.h"

static uint32_t joint_dofs(uint32_t t) {
    switch (t) {
        case ORC_JOINT_REVOLUTE: case ORC_JOINT_PRISMATIC: return 1u;
        case ORC_JOINT_FLOATING: return 6u;
        case ORC_JOINT_SPHERICAL: return 3u;
        default: return 0u;
    }
}

/* cuda_vec_ops.cuh ContactTangentBasis */
static void tangent_basis(v3 normal, v3 *t1, v3 *t2) {
    float ls = vdot(normal, normal);
    v3 n = ls > 1.0e-10f ? vscale(normal, rsq(ls)) : V3(0, 0, 1);
    v3 ref = V3(1, 0, 0);
    if (fabsf(n.x) > 0.9f) ref = V3(0, 1, 0);
    float proj = vdot(ref, n);
    v3 ta = V3(ref.x - proj * n.x, ref.y - proj * n.y, ref.z - proj * n.z);
    float l2 = vdot(ta, ta);
    if (l2 > 1.0e-12f) ta = vscale(ta, rsq(l2)); else ta = V3(1, 0, 0);
    *t1 = ta; *t2 = vcross(n, ta);
}

/* articulation_types.cuh:193-238 AccumulateChainJointForce with tau = 0, walked leaf to root
 * (assemble_rows.cu:122-169 ComputeContactChainJacobianKernel). */
static void chain_jacobian(const orc_model *m, const orc_env *e, uint32_t link, v3 point, v3 f, float *out) {
    for (uint32_t k = 0; k < m->ndof; ++k) out[k] = 0.0f;
    uint32_t l = link;
    while (l != ORC_NOLINK) {
        const uint32_t type = m->jtype[l];
        if (joint_dofs(type) != 0u) {
            const uint32_t d = m->link_dof[l];
            if (type == ORC_JOINT_FLOATING) {
                quat br = qld(e->base_pose + 3);
                v3 lever = vsub(point, v3ld(e->base_pose));
                v3 ex = qrot(br, V3(1, 0, 0)), ey = qrot(br, V3(0, 1, 0)), ez = qrot(br, V3(0, 0, 1));
                const float ang[3] = {vdot(vcross(ex, lever), f) + 0.0f, vdot(vcross(ey, lever), f) + 0.0f, vdot(vcross(ez, lever), f) + 0.0f};
                const float lin[3] = {vdot(ex, f), vdot(ey, f), vdot(ez, f)};
                for (uint32_t b = 0; b < 3u; ++b) { out[d + b] += ang[b]; out[d + 3u + b] += lin[b]; }
            } else {
                v3 axis_w = qrot(qld(e->link_pose + 7 * l + 3), v3ld(m->axis + 3 * l));
                float entry;
                if (type == ORC_JOINT_PRISMATIC) entry = vdot(axis_w, f);
                else entry = vdot(vcross(axis_w, vsub(point, v3ld(e->link_pose + 7 * l))), f) + 0.0f;
                out[d] += entry;
            }
        }
        l = m->parent[l];
    }
}

static void resolve_side(const orc_model *m, uint32_t body, orc_side *s, uint32_t *link) {
    /* collidable_owner.hpp:28-62 */
    *link = ORC_NOLINK;
    s->index = ORC_NOLINK;
    if (m->body_id[body] < 0) { s->kind = ORC_SIDE_STATIC; return; }
    if (m->body_to_link[body] == ORC_NOLINK) { s->kind = ORC_SIDE_RIGID; s->index = body; return; }
    s->kind = ORC_SIDE_ARTIC; s->index = 0u; *link = m->body_to_link[body];
}

static orc_row *new_row(orc_env *e) {
    orc_row *r = &e->rows[e->nrows++];
    memset(r, 0, sizeof(*r));
    r->a.kind = r->b.kind = ORC_SIDE_STATIC; r->a.index = r->b.index = ORC_NOLINK;
    r->contact_slot = r->contact_point = ORC_NOLINK; r->link = ORC_NOLINK;
    return r;
}
static float *new_jac(const orc_model *m, orc_env *e, uint32_t row_index, int side) {
    return e->jac_pool + ((size_t)row_index * 2u + (size_t)side) * m->ndof;
}

static void fill_sides(const orc_model *m, orc_env *e, orc_row *r, uint32_t ri, const orc_side *sa, const orc_side *sb,
                       uint32_t la, uint32_t lb, v3 dir, v3 point, v3 com_a, v3 com_b) {
    r->a = *sa; r->b = *sb;
    v3st(r->a.jlin, dir); v3st(r->b.jlin, vneg(dir));
    v3st(r->a.jang, V3(0, 0, 0)); v3st(r->b.jang, V3(0, 0, 0));
    if (sa->kind == ORC_SIDE_RIGID) v3st(r->a.jang, vcross(vsub(point, com_a), dir));
    if (sb->kind == ORC_SIDE_RIGID) v3st(r->b.jang, vcross(vsub(point, com_b), vneg(dir)));
    if (sa->kind == ORC_SIDE_ARTIC) { r->ja = new_jac(m, e, ri, 0); chain_jacobian(m, e, la, point, dir, r->ja); }
    if (sb->kind == ORC_SIDE_ARTIC) { r->jb = new_jac(m, e, ri, 1); chain_jacobian(m, e, lb, point, vneg(dir), r->jb); }
    /* assemble_rows.cu:172-186: one articulation on both sides keeps the net chain on side a */
    if (r->ja && r->jb) { for (uint32_t k = 0; k < m->ndof; ++k) { r->ja[k] += r->jb[k]; r->jb[k] = 0.0f; } }
}

/* assemble_rows.cu:406-801 (speculative law, condim 3) then 805-971 joint rows */
void orc_assemble_rows(const orc_model *m, orc_env *e) {
    const float dt = m->cfg.dt;
    const int position_pass = m->cfg.pos_iters > 0u;
    e->nrows = 0;
    for (uint32_t s = 0; s < m->cfg.max_contacts; ++s) {
        const uint32_t pts = e->ccount[s];
        if (pts == 0u) continue;
        const uint32_t a = e->pairs[2 * s], b = e->pairs[2 * s + 1];
        orc_side sa, sb; uint32_t la, lb;
        memset(&sa, 0, sizeof sa); memset(&sb, 0, sizeof sb);
        resolve_side(m, a, &sa, &la); resolve_side(m, b, &sb, &lb);
        v3 com_a = V3(0, 0, 0), com_b = V3(0, 0, 0);
        if (sa.kind == ORC_SIDE_RIGID) com_a = vadd(v3ld(e->body_pose + 7 * a), qrot(qld(e->body_pose + 7 * a + 3), v3ld(m->inertial_pos + 3 * a)));
        if (sb.kind == ORC_SIDE_RIGID) com_b = vadd(v3ld(e->body_pose + 7 * b), qrot(qld(e->body_pose + 7 * b + 3), v3ld(m->inertial_pos + 3 * b)));
        /* contact_filter.hpp:88-140: equal priority, non-geometric mixing takes the larger coefficient */
        const float mu = m->mu[a] > m->mu[b] ? m->mu[a] : m->mu[b];
        const uint32_t base = e->nrows;
        for (uint32_t k = 0; k < 3u * pts; ++k) new_row(e);
        for (uint32_t p = 0; p < pts; ++p) {
            const uint32_t at = s * 4u + p;
            v3 raw = v3ld(e->cnormal + 3 * at), point = v3ld(e->cpoint + 3 * at);
            float len = sqrtf(raw.x * raw.x + raw.y * raw.y + raw.z * raw.z);
            v3 n = len < 1e-12f ? V3(0, 0, 0) : V3(raw.x / len, raw.y / len, raw.z / len);
            v3 t0, t1; tangent_basis(raw, &t0, &t1);
            const float cd = e->cdepth[at];
            /* assemble_rows.cu:702-712 rounding reserve of the projected endpoints */
            v3 ext = V3(fabsf(point.x) + fabsf(n.x * cd), fabsf(point.y) + fabsf(n.y * cd), fabsf(point.z) + fabsf(n.z * cd));
            const double gamma = 3.0 * (double)FLT_EPSILON / (1.0 - 3.0 * (double)FLT_EPSILON);
            const double roundoff = gamma * (fabs((double)n.x) * (fabs((double)ext.x) + fabs((double)ext.x)) +
                                             fabs((double)n.y) * (fabs((double)ext.y) + fabs((double)ext.y)) +
                                             fabs((double)n.z) * (fabs((double)ext.z) + fabs((double)ext.z)));
            const float clearance = roundoff > 0.0 ? nextafterf((float)roundoff, FLT_MAX) : 0.0f;
            const float depth = cd + clearance;
            const uint32_t ri[3] = {base + p, base + pts + p, base + 2u * pts + p};
            const v3 dirs[3] = {n, t0, t1};
            for (int k = 0; k < 3; ++k) {
                orc_row *r = &e->rows[ri[k]];
                r->group_first = base; r->group_normal_count = pts;
                r->mu = mu; r->mu2 = mu; r->tag = 0u;
                r->contact_slot = s; r->contact_point = p;
                fill_sides(m, e, r, ri[k], &sa, &sb, la, lb, dirs[k], point, com_a, com_b);
                if (k == 0) {
                    r->flags = ORC_ROW_ACTIVE | ORC_ROW_CONTACT_NORMAL | ORC_ROW_BLOCK_NORMAL | ORC_ROW_SPECULATIVE;
                    r->penetration = depth;
                    r->rhs = (fminf(depth, 0.0f) + (position_pass ? 0.0f
                              : fminf(fmaxf(cd, 0.0f), m->cfg.overlap_recovery_velocity * dt))) / (dt * dt);
                    r->lower = 0.0f; r->upper = FLT_MAX;
                } else {
                    r->flags = ORC_ROW_ACTIVE | ORC_ROW_BLOCK_TANGENT;
                    r->lower = -FLT_MAX; r->upper = FLT_MAX;
                }
            }
        }
    }
    /* joint limit rows, assemble_rows.cu:805-882 */
    for (uint32_t l = 0; l < m->L; ++l) for (uint32_t side = 0; side < 2u; ++side) {
        if (joint_dofs(m->jtype[l]) != 1u || !(m->limit_flags[l] & (1u << side))) continue;
        orc_row *r = new_row(e);
        const uint32_t ri = (uint32_t)(r - e->rows);
        const float bound = side == 0u ? m->limit_lower[l] : m->limit_upper[l];
        const float dist = side == 0u ? e->q[l] - bound : bound - e->q[l];
        const float target = -(position_pass ? fmaxf(dist, 0.0f) : dist) / dt;
        r->flags = ORC_ROW_ACTIVE | (side == 0u ? ORC_ROW_LIMIT_LOWER : ORC_ROW_LIMIT_UPPER);
        r->group_first = ri; r->group_normal_count = 1u;
        r->rhs = fminf(target, m->cfg.baumgarte_max_velocity) / dt;
        r->lower = 0.0f; r->upper = FLT_MAX;
        r->a.kind = ORC_SIDE_ARTIC; r->a.index = 0u;
        r->ja = new_jac(m, e, ri, 0);
        for (uint32_t k = 0; k < m->ndof; ++k) r->ja[k] = 0.0f;
        r->ja[m->link_dof[l]] = side == 0u ? 1.0f : -1.0f;
        r->penetration = fmaxf(-dist, 0.0f);
        /* an authored limit row starts from the multiplier the last step's solve left in its slot (assemble_rows.cu:826-879
         * clears lambda only for links without that limit, and the per-step clear :366-383 covers the contact rows alone) */
        r->lambda = e->limit_lambda[2u * l + side];
        r->tag = 1u; r->link = l;
    }
    /* joint dry friction rows, assemble_rows.cu:886-934 */
    for (uint32_t l = 0; l < m->L; ++l) {
        const float fr = m->frictionloss[l];
        if (joint_dofs(m->jtype[l]) != 1u || !(fr > 0.0f)) continue;
        orc_row *r = new_row(e);
        const uint32_t ri = (uint32_t)(r - e->rows);
        r->flags = ORC_ROW_ACTIVE | ORC_ROW_VELOCITY_ONLY;
        r->group_first = ri; r->group_normal_count = 1u;
        r->lower = -fr * dt; r->upper = fr * dt;
        r->a.kind = ORC_SIDE_ARTIC; r->a.index = 0u;
        r->ja = new_jac(m, e, ri, 0);
        for (uint32_t k = 0; k < m->ndof; ++k) r->ja[k] = 0.0f;
        r->ja[m->link_dof[l]] = 1.0f;
        r->tag = 2u; r->link = l;
    }
    /* drive rows, assemble_rows.cu:938-971 */
    for (uint32_t l = 0; l < m->L; ++l) {
        if (joint_dofs(m->jtype[l]) != 1u) continue;
        const float effort = fminf(fmaxf(e->drive_command[l], e->drive_lower[l]), e->drive_upper[l]);
        if (effort == 0.0f) continue;
        orc_row *r = new_row(e);
        const uint32_t ri = (uint32_t)(r - e->rows);
        r->flags = ORC_ROW_ACTIVE | ORC_ROW_VELOCITY_ONLY;
        r->group_first = ri; r->group_normal_count = 1u;
        r->a.kind = ORC_SIDE_ARTIC; r->a.index = 0u;
        r->ja = new_jac(m, e, ri, 0);
        for (uint32_t k = 0; k < m->ndof; ++k) r->ja[k] = 0.0f;
        r->ja[m->link_dof[l]] = 1.0f;
        r->lower = r->upper = effort * dt;
        r->lambda = r->lower;
        r->tag = 3u; r->link = l;
    }
}

/* Warm start, phase 0 (assemble_rows.cu:1228-1273 + contact_cache.cuh BuildIndex): a current point takes the
 * multipliers of the cached point with the same (pair, feature) identity whose age is below the decay bound,
 * when the normals agree; only the first current point of an identity matches. The material hash is equal for
 * every contact here (one law, one cone), so it does not enter the key. */
void orc_warm_start_prepare(const orc_model *m, orc_env *e) {
    const uint32_t npts = m->cfg.max_contacts * 4u;
    for (uint32_t r = 0; r < e->nrows; ++r) {
        orc_row *row = &e->rows[r];
        if (row->tag != 0u || !(row->flags & ORC_ROW_BLOCK_NORMAL)) continue;
        const uint32_t at = row->contact_slot * 4u + row->contact_point;
        int first = 1;
        for (uint32_t s = 0; s < row->contact_slot * 4u + row->contact_point && first; ++s) {
            if ((s & 3u) < e->ccount[s >> 2] && e->cid_pair[s] == e->cid_pair[at] && e->cid_feature[s] == e->cid_feature[at]) first = 0;
        }
        if (!first) continue;
        const orc_cache_entry *match = NULL;
        for (uint32_t c = 0; c < npts; ++c) {
            const orc_cache_entry *en = &e->cache[c];
            if (en->valid && en->age < 2u && en->pair == e->cid_pair[at] && en->feature == e->cid_feature[at]) { match = en; break; }
        }
        if (!match) continue;
        v3 n = v3ld(e->cnormal + 3 * at), cn = v3ld(match->normal);
        if (!(vdot(n, cn) > 0.25f)) continue;
        v3 ot1, ot2, t1, t2;
        tangent_basis(cn, &ot1, &ot2);
        tangent_basis(n, &t1, &t2);
        v3 old = vadd(vscale(ot1, match->lambda[1]), vscale(ot2, match->lambda[2]));
        const uint32_t pts = row->group_normal_count;
        row->lambda = fmaxf(match->lambda[0], 0.0f);
        e->rows[r + pts].lambda = vdot(old, t1);
        e->rows[r + 2u * pts].lambda = vdot(old, t2);
    }
}

/* Warm start, phase 1 (assemble_rows.cu:1323-1391 RebuildContactCacheKernel): current points own their cache
 * point with age 0; unmatched cached identities of age 0 survive one more step in the free points. */
void orc_warm_start_commit(const orc_model *m, orc_env *e) {
    const uint32_t npts = m->cfg.max_contacts * 4u;
    orc_cache_entry *next = e->cache_next;
    memset(next, 0, sizeof(orc_cache_entry) * npts);
    uint8_t owner[4096];
    memset(owner, 0, sizeof owner);
    /* owners: the first current point of each identity */
    for (uint32_t r = 0; r < e->nrows; ++r) {
        const orc_row *row = &e->rows[r];
        if (row->tag != 0u || !(row->flags & ORC_ROW_CONTACT_NORMAL)) continue;
        const uint32_t at = row->contact_slot * 4u + row->contact_point;
        int first = 1;
        for (uint32_t s = 0; s < at && first; ++s)
            if ((s & 3u) < e->ccount[s >> 2] && e->cid_pair[s] == e->cid_pair[at] && e->cid_feature[s] == e->cid_feature[at]) first = 0;
        if (!first) continue;
        const uint32_t pts = row->group_normal_count;
        orc_cache_entry *en = &next[at];
        en->valid = 1u; en->age = 0u;
        en->pair = e->cid_pair[at]; en->feature = e->cid_feature[at];
        en->lambda[0] = row->lambda; en->lambda[1] = e->rows[r + pts].lambda; en->lambda[2] = e->rows[r + 2u * pts].lambda; en->lambda[3] = 0.0f;
        memcpy(en->normal, e->cnormal + 3 * at, 12);
        owner[at] = 1u;
    }
    /* retained: cached identities with no current twin and age < decay_steps - 1, first of their identity */
    uint32_t free_at = 0;
    for (uint32_t c = 0; c < npts; ++c) {
        const orc_cache_entry *en = &e->cache[c];
        if (!en->valid || en->age >= 1u) continue;
        int twin = 0;
        for (uint32_t s = 0; s < npts && !twin; ++s)
            if ((s & 3u) < e->ccount[s >> 2] && e->cid_pair[s] == en->pair && e->cid_feature[s] == en->feature) twin = 1;
        for (uint32_t d = 0; d < c && !twin; ++d)
            if (e->cache[d].valid && e->cache[d].pair == en->pair && e->cache[d].feature == en->feature) twin = 1;
        if (twin) continue;
        while (free_at < npts && owner[free_at]) ++free_at;
        if (free_at >= npts) break;
        next[free_at] = *en;
        next[free_at].age = en->age + 1u;
        ++free_at;
    }
    e->cache_next = e->cache; e->cache = next;
}
