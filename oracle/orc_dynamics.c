/* Oracle (test infrastructure): kinematics, drives, joint-space dynamics, integration.
 * Restates the reference's src/phi/backend_cuda/ops/articulation.cu, articulation_mass.cuh
 * and kinematics.cuh stage by stage on one env. */
#include "orc.h"
#include "orc_math.h"

static uint32_t joint_dofs(uint32_t t) {
    /* articulation_types.cuh:101-114 */
    switch (t) {
        case ORC_JOINT_REVOLUTE: case ORC_JOINT_PRISMATIC: return 1u;
        case ORC_JOINT_FLOATING: return 6u;
        case ORC_JOINT_SPHERICAL: return 3u;
        default: return 0u;
    }
}

/* kinematics.cuh:25-42 JointRelativeFrame (revolute / prismatic / fixed / floating) */
static void joint_relative_frame(const orc_model *m, const orc_env *e, uint32_t l, float *out) {
    v3 axis = v3ld(m->axis + 3 * l);
    float ls = vdot(axis, axis);
    axis = ls > 1.0e-12f ? vscale(axis, rsq(ls)) : V3(0, 0, 0);
    v3 pos = vadd(v3ld(m->local_pos + 3 * l), v3ld(m->parent_offset + 3 * l));
    quat rot = qld(m->local_quat + 4 * l);
    if (m->jtype[l] == ORC_JOINT_REVOLUTE) {
        float half = 0.5f * e->q[l], s = sinf(half);
        quat turn = Q4(cosf(half), axis.x * s, axis.y * s, axis.z * s);
        rot = qnorm_le(qmul(rot, turn), 1.0e-12f);
    } else if (m->jtype[l] == ORC_JOINT_PRISMATIC) {
        pos = vadd(pos, qrot(rot, vscale(axis, e->q[l])));
    }
    v3st(out, pos); qst(out + 3, rot);
}

/* articulation.cu:1561-1596 UpdateWorldLinkPosesKernel */
void orc_fk(const orc_model *m, orc_env *e) {
    for (uint32_t l = 0; l < m->L; ++l) {   /* parents precede children in link order */
        float rel[7];
        joint_relative_frame(m, e, l, rel);
        if (m->parent[l] == ORC_NOLINK) {
            if (m->jtype[l] == ORC_JOINT_FLOATING) memcpy(e->link_pose + 7 * l, e->base_pose, 28);
            else memcpy(e->link_pose + 7 * l, rel, 28);
        } else {
            pose_compose(e->link_pose + 7 * m->parent[l], rel, e->link_pose + 7 * l);
        }
    }
}

/* articulation.cu:836-940 ApplyAffineDriveKernel, control mode 0 (implicit PD position);
 * joint_force_limit = 0, joint gravity force = 0 (no actuator gravity compensation). */
void orc_apply_drives(const orc_model *m, orc_env *e) {
    const float dt = m->cfg.dt;
    for (uint32_t l = 0; l < m->L; ++l) {
        e->drive_command[l] = e->drive_dissipation[l] = 0.0f;
        e->drive_lower[l] = e->drive_upper[l] = 0.0f;
        e->tau[l] = 0.0f;
        if (joint_dofs(m->jtype[l]) != 1u) continue;
        const uint32_t mode = m->cfg.control_mode;
        const int inverse_dynamics = mode == 3u || mode == 4u;       /* articulation.cu:848-849 */
        const int position_control = mode == 0u || inverse_dynamics, velocity_control = mode == 2u;
        if ((position_control && (!isfinite(e->drive_target[l]) || !isfinite(e->kp[l]) || e->kp[l] < 0.0f ||
                                  !isfinite(e->kd[l]) || e->kd[l] < 0.0f)) ||
            ((position_control || velocity_control) && !isfinite(e->vel_target[l])) ||
            (velocity_control && (!isfinite(e->kp[l]) || e->kp[l] < 0.0f)) ||
            (mode == 3u && !isfinite(e->acc_target[l])) ||
            (mode == 5u && !isfinite(e->noload_speed[l]))) {
            e->status |= ORC_STATUS_CONTROL_FAILURE;
            continue;
        }
        const float velocity = e->qdot[l];
        const float limit = e->force_limit[l];
        float lower = limit > 0.0f ? -limit : -FLT_MAX;
        float upper = limit > 0.0f ? limit : FLT_MAX;
        float damping = 0.0f, bias = 0.0f;
        if (inverse_dynamics) {
            /* articulation.cu:899-901: no affine term here; the controller below writes the command */
        } else if (position_control) {
            damping = e->kd[l] + dt * e->kp[l];
            bias = e->kp[l] * (e->drive_target[l] - e->q[l]) + damping * e->vel_target[l];
        } else if (velocity_control) {
            damping = e->kp[l];
            bias = damping * e->vel_target[l];
        } else {
            bias = e->drive_target[l];             /* torque, actuator: the target field carries the commanded effort */
            if (mode == 5u && limit > 0.0f && e->noload_speed[l] > 0.0f) {
                /* signed torque-speed envelope, articulation.cu:892-898 */
                const float speed_bias = limit * velocity / e->noload_speed[l];
                lower = fminf(fmaxf(-limit - speed_bias, -limit), limit);
                upper = fminf(fmaxf(limit - speed_bias, -limit), limit);
            }
        }
        const float effort = bias - damping * velocity;
        const int saturated = effort < lower || effort > upper;
        if (saturated) {
            bias = effort;
            damping = 0.0f;
        } else {
            lower += damping * velocity;
            upper += damping * velocity;
        }
        const float ff = e->feedforward[l];
        if (!isfinite(bias) || !isfinite(damping) || damping < 0.0f || !isfinite(limit) ||
            !isfinite(ff) || !isfinite(velocity) || !isfinite(e->q[l])) {
            e->status |= ORC_STATUS_CONTROL_FAILURE;
            continue;
        }
        if (inverse_dynamics) {                    /* articulation.cu:932-939: the bounds are the plain force limit */
            lower = limit > 0.0f ? -limit : -FLT_MAX;
            upper = limit > 0.0f ? limit : FLT_MAX;
        }
        e->drive_command[l] = bias;
        e->drive_dissipation[l] = damping;
        e->drive_lower[l] = lower;
        e->drive_upper[l] = upper;
        e->tau[l] = inverse_dynamics ? 0.0f : ff;
    }
}

/* articulation.cu:1193-1230 FactorControlMass / SolveControlMass: L D L^T of the actuated block with double accumulators */
static int factor_control_mass(float *a, uint32_t n, uint32_t stride, float *diagonal) {
    for (uint32_t j = 0; j < n; ++j) {
        double pivot = a[j * stride + j];
        for (uint32_t k = 0; k < j; ++k) { const double v = a[j * stride + k]; pivot -= v * v * diagonal[k]; }
        if (!(pivot > 0.0) || !isfinite(pivot)) return 0;
        diagonal[j] = (float)pivot;
        for (uint32_t i = j + 1u; i < n; ++i) {
            double v = a[i * stride + j];
            for (uint32_t k = 0; k < j; ++k) v -= (double)a[i * stride + k] * a[j * stride + k] * diagonal[k];
            a[i * stride + j] = (float)(v / pivot);
        }
    }
    return 1;
}
static void solve_control_mass(const float *f, const float *diagonal, uint32_t n, uint32_t stride, const float *rhs, float *x) {
    for (uint32_t i = 0; i < n; ++i) {
        double v = rhs[i];
        for (uint32_t j = 0; j < i; ++j) v -= (double)f[i * stride + j] * x[j];
        x[i] = (float)v;
    }
    for (uint32_t i = 0; i < n; ++i) x[i] /= diagonal[i];
    for (uint32_t ii = n; ii > 0u; --ii) {
        const uint32_t i = ii - 1u;
        double v = x[i];
        for (uint32_t j = i + 1u; j < n; ++j) v -= (double)f[j * stride + i] * x[j];
        x[i] = (float)v;
    }
}

/* articulation.cu:1234-1288 InvertTaskResponse: symmetric pseudoinverse by cyclic Jacobi rotations; directions whose
 * eigenvalue is within 8 eps of the largest are dropped */
static void invert_task_response(float *a, uint32_t n, float *inverse) {
    float vec[36];
    memset(vec, 0, sizeof vec);
    for (uint32_t i = 0; i < n; ++i) vec[i * 6u + i] = 1.0f;
    for (uint32_t sweep = 0; sweep < 24u; ++sweep) {
        int changed = 0;
        for (uint32_t p = 0; p < n; ++p) for (uint32_t q = p + 1u; q < n; ++q) {
            const float app = a[p * 6u + p], aqq = a[q * 6u + q], apq = a[p * 6u + q];
            if (fabsf(apq) <= FLT_EPSILON * (fabsf(app) + fabsf(aqq))) continue;
            changed = 1;
            const double theta = ((double)aqq - app) / (2.0 * apq);
            const float tangent = (float)(copysign(1.0, theta) / (fabs(theta) + sqrt(1.0 + theta * theta)));
            const float cosine = rsq(1.0f + tangent * tangent);
            const float sine = tangent * cosine;
            for (uint32_t k = 0; k < n; ++k) {
                if (k != p && k != q) {
                    const float kp = a[k * 6u + p], kq = a[k * 6u + q];
                    a[k * 6u + p] = a[p * 6u + k] = cosine * kp - sine * kq;
                    a[k * 6u + q] = a[q * 6u + k] = sine * kp + cosine * kq;
                }
                const float vp = vec[k * 6u + p], vq = vec[k * 6u + q];
                vec[k * 6u + p] = cosine * vp - sine * vq;
                vec[k * 6u + q] = sine * vp + cosine * vq;
            }
            a[p * 6u + p] = app - tangent * apq;
            a[q * 6u + q] = aqq + tangent * apq;
            a[p * 6u + q] = a[q * 6u + p] = 0.0f;
        }
        if (!changed) break;
    }
    float largest = 0.0f;
    for (uint32_t i = 0; i < n; ++i) largest = fmaxf(largest, a[i * 6u + i]);
    const float tolerance = largest * (8.0f * FLT_EPSILON);
    for (uint32_t r = 0; r < n; ++r) for (uint32_t c = 0; c < n; ++c) {
        double v = 0.0;
        for (uint32_t k = 0; k < n; ++k) {
            const float eigenvalue = a[k * 6u + k];
            if (eigenvalue > tolerance) v += (double)vec[r * 6u + k] * vec[c * 6u + k] / eigenvalue;
        }
        inverse[r * 6u + c] = (float)v;
    }
}
/* articulation.cu:1300-1313 TaskOrientationError: rotation vector from the current to the desired orientation */
static v3 task_orientation_error(quat desired, quat current) {
    current = qnorm_le(current, 1.0e-12f); desired = qnorm_le(desired, 1.0e-12f);
    const quat err = qmul(desired, Q4(current.w, -current.x, -current.y, -current.z));
    const float sign = err.w < 0.0f ? -1.0f : 1.0f;
    const float length = sqrtf(err.x * err.x + err.y * err.y + err.z * err.z);
    const float scale = length > 1.0e-7f ? sign * 2.0f * atan2f(length, fabsf(err.w)) / length : sign * 2.0f;
    return V3(err.x * scale, err.y * scale, err.z * scale);
}

/* Operational-space control, articulation.cu:1419-1550 (the Osc branch of ApplyDynamicsDriveKernel).  J is the 6 x n
 * Jacobian of the task frame (linear rows first), B = J M^-1 S^T its response to the actuators, H the actuated inertia
 * of the computed-torque branch.  The task force F = (B H B^T)^+ (kp x_err - kd v - a_free - B (bias + damping + posture))
 * acts through H B^T; joints on the chain from the task link to the root hold their posture through the nullspace gains,
 * joints off the chain through their own drive gains. */
static void osc_command(const orc_model *m, orc_env *e, uint32_t active, const uint32_t *links, const uint32_t *dofs,
                        const float *mass, const float *bias, uint32_t stride) {
    const uint32_t n = m->ndof, task_link = m->cfg.task_link;
    static _Thread_local float jac[6 * ORC_MAX_DOF], response[6 * ORC_MAX_DOF], task_map[6 * ORC_MAX_DOF];
    uint32_t chain[ORC_MAX_DOF];
    float solution[ORC_MAX_DOF], rhs[ORC_MAX_DOF], posture[ORC_MAX_DOF];
    float local_task[7];
    memcpy(local_task, e->task_frame, sizeof local_task);
    qst(local_task + 3, qnorm_le(qld(local_task + 3), 1.0e-12f));
    float task_pose[7];
    pose_compose(e->link_pose + 7 * task_link, local_task, task_pose);
    memset(jac, 0, sizeof(float) * 6u * stride);
    memset(chain, 0, sizeof chain);
    for (uint32_t walk = task_link; walk != ORC_NOLINK; walk = m->parent[walk]) {
        const uint32_t type = m->jtype[walk], dof = m->link_dof[walk];
        const v3 lever = vsub(v3ld(task_pose), v3ld(e->link_pose + 7 * walk));
        if (type == ORC_JOINT_FLOATING) {
            const v3 basis[3] = {V3(1, 0, 0), V3(0, 1, 0), V3(0, 0, 1)};
            for (uint32_t c = 0; c < 3u; ++c) {
                const v3 axis = qrot(qld(e->base_pose + 3), basis[c]);
                const v3 lin = vcross(axis, lever);
                jac[dof + c] = lin.x; jac[stride + dof + c] = lin.y; jac[2u * stride + dof + c] = lin.z;
                jac[3u * stride + dof + c] = axis.x; jac[4u * stride + dof + c] = axis.y; jac[5u * stride + dof + c] = axis.z;
                jac[dof + 3u + c] = axis.x; jac[stride + dof + 3u + c] = axis.y; jac[2u * stride + dof + 3u + c] = axis.z;
                jac[3u * stride + dof + 3u + c] = 0.0f; jac[4u * stride + dof + 3u + c] = 0.0f; jac[5u * stride + dof + 3u + c] = 0.0f;
            }
        } else if (joint_dofs(type) == 1u) {
            const v3 axis = qrot(qld(e->link_pose + 7 * walk + 3), v3ld(m->axis + 3 * walk));
            const int revolute = type == ORC_JOINT_REVOLUTE;
            const v3 lin = revolute ? vcross(axis, lever) : axis, ang = revolute ? axis : V3(0, 0, 0);
            jac[dof] = lin.x; jac[stride + dof] = lin.y; jac[2u * stride + dof] = lin.z;
            jac[3u * stride + dof] = ang.x; jac[4u * stride + dof] = ang.y; jac[5u * stride + dof] = ang.z;
            chain[dof] = 1u;
        }
    }
    const quat desired = qld(e->task_rotation);
    const float rotation_norm = desired.w * desired.w + desired.x * desired.x + desired.y * desired.y + desired.z * desired.z;
    const uint32_t rows = rotation_norm > 1.0e-12f ? 6u : 3u;
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t d = 0; d < n; ++d) solution[d] = jac[r * stride + d];
        orc_solve_mass(e->Mfactor, solution, n);
        for (uint32_t c = 0; c < active; ++c) response[r * stride + c] = solution[dofs[c]];
    }
    for (uint32_t r = 0; r < rows; ++r) for (uint32_t c = 0; c < active; ++c) {
        double v = 0.0;
        for (uint32_t a = 0; a < active; ++a) v += (double)mass[c * stride + a] * response[r * stride + a];
        task_map[r * stride + c] = (float)v;
    }
    float metric[36], inverse_metric[36];
    memset(metric, 0, sizeof metric); memset(inverse_metric, 0, sizeof inverse_metric);
    for (uint32_t r = 0; r < rows; ++r) for (uint32_t c = 0; c < rows; ++c) {
        double v = 0.0;
        for (uint32_t a = 0; a < active; ++a) v += (double)response[r * stride + a] * task_map[c * stride + a];
        metric[r * 6u + c] = (float)v;
    }
    invert_task_response(metric, rows, inverse_metric);
    const float *vel = e->link_vel + 6 * task_link, *acc = e->link_acc + 6 * task_link;
    const v3 omega = V3(vel[0], vel[1], vel[2]), linear = V3(vel[3], vel[4], vel[5]);
    const v3 alpha = V3(acc[0], acc[1], acc[2]), linear_accel = V3(acc[3], acc[4], acc[5]);
    const quat rotation = qld(e->link_pose + 7 * task_link + 3);
    const v3 offset = v3ld(local_task);
    const v3 task_velocity = qrot(rotation, vadd(linear, vcross(omega, offset)));
    const v3 task_angular = qrot(rotation, omega);
    const v3 task_accel = vadd(qrot(rotation, vadd(vadd(linear_accel, vcross(omega, linear)),
                                                   vadd(vcross(alpha, offset), vcross(omega, vcross(omega, offset))))),
                               V3(m->cfg.gravity[0], m->cfg.gravity[1], m->cfg.gravity[2]));
    const v3 task_angular_accel = qrot(rotation, alpha);
    const v3 position_error = vsub(v3ld(e->task_target), v3ld(task_pose));
    const v3 orientation_error = rows == 6u ? task_orientation_error(desired, qld(task_pose + 3)) : V3(0, 0, 0);
    const float kp = e->kp[task_link], kd = e->kd[task_link];
    float task_rhs[6] = {kp * position_error.x - kd * task_velocity.x - task_accel.x,
                         kp * position_error.y - kd * task_velocity.y - task_accel.y,
                         kp * position_error.z - kd * task_velocity.z - task_accel.z,
                         kp * orientation_error.x - kd * task_angular.x - task_angular_accel.x,
                         kp * orientation_error.y - kd * task_angular.y - task_angular_accel.y,
                         kp * orientation_error.z - kd * task_angular.z - task_angular_accel.z};
    for (uint32_t c = 0; c < active; ++c) {
        const uint32_t l = links[c];
        rhs[c] = chain[dofs[c]] ? e->null_kp * (e->drive_target[l] - e->q[l]) + e->null_kd * (e->vel_target[l] - e->qdot[l]) : 0.0f;
    }
    for (uint32_t r = 0; r < active; ++r) {
        double v = 0.0;
        for (uint32_t c = 0; c < active; ++c) v += (double)mass[r * stride + c] * rhs[c];
        const uint32_t l = links[r];
        if (!chain[dofs[r]]) v += e->kp[l] * (e->drive_target[l] - e->q[l]) + e->kd[l] * (e->vel_target[l] - e->qdot[l]);
        posture[r] = (float)v;
    }
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t a = 0; a < active; ++a)
            task_rhs[r] -= response[r * stride + a] * (bias[a] + m->damping[links[a]] * e->qdot[links[a]] + posture[a]);
    float task_force[6] = {0, 0, 0, 0, 0, 0};
    for (uint32_t r = 0; r < rows; ++r) for (uint32_t c = 0; c < rows; ++c) task_force[r] += inverse_metric[r * 6u + c] * task_rhs[c];
    for (uint32_t a = 0; a < active; ++a) {
        double v = bias[a] + posture[a];
        for (uint32_t r = 0; r < rows; ++r) v += (double)task_map[r * stride + a] * task_force[r];
        e->drive_command[links[a]] = (float)v;
    }
}

/* Computed-torque control, articulation.cu:1315-1418 (ApplyDynamicsDriveKernel, ComputedTorque branch).  With S the
 * selector of the scalar joints, H = (S M^-1 S^T)^-1 is the inertia the actuators see (a floating base's reaction
 * included); the command is H (a* + kp (q* - q) + kd (qd* - qd)) plus the compensation of the force-free acceleration,
 * passive joint damping left out of it. */
void orc_apply_dynamics_drives(const orc_model *m, orc_env *e) {
    const uint32_t L = m->L, n = m->ndof;
    uint32_t links[ORC_MAX_DOF], dofs[ORC_MAX_DOF], active = 0u;
    if (m->cfg.control_mode == 4u && m->cfg.task_link >= L) { e->status |= ORC_STATUS_CONTROL_FAILURE; return; }
    for (uint32_t l = 0; l < L; ++l)
        if (joint_dofs(m->jtype[l]) == 1u && e->drive_lower[l] == 0.0f && e->drive_upper[l] == 0.0f) return;     /* a rejected drive */
    if (m->cfg.control_mode == 4u) {           /* articulation.cu:1341-1360 */
        const uint32_t tl = m->cfg.task_link;
        int ok = isfinite(e->kp[tl]) && e->kp[tl] >= 0.0f && isfinite(e->kd[tl]) && e->kd[tl] >= 0.0f &&
                 isfinite(e->null_kp) && e->null_kp >= 0.0f && isfinite(e->null_kd) && e->null_kd >= 0.0f;
        for (int k = 0; k < 3; ++k) ok &= isfinite(e->task_target[k]);
        for (int k = 0; k < 4; ++k) ok &= isfinite(e->task_rotation[k]);
        for (int k = 0; k < 7; ++k) ok &= isfinite(e->task_frame[k]);
        if (!ok) { e->status |= ORC_STATUS_CONTROL_FAILURE; return; }
    }
    for (uint32_t l = 0; l < L; ++l) {
        if (joint_dofs(m->jtype[l]) != 1u) continue;
        links[active] = l; dofs[active] = m->link_dof[l];
        e->tau[l] = e->feedforward[l];
        ++active;
    }
    if (active == 0u) return;
    static _Thread_local float factor[ORC_MAX_DOF * ORC_MAX_DOF], mass[ORC_MAX_DOF * ORC_MAX_DOF];
    float diagonal[ORC_MAX_DOF], rhs[ORC_MAX_DOF], solution[ORC_MAX_DOF], bias[ORC_MAX_DOF];
    const uint32_t stride = n;
    for (uint32_t c = 0; c < active; ++c) {
        for (uint32_t d = 0; d < n; ++d) solution[d] = d == dofs[c] ? 1.0f : 0.0f;
        orc_solve_mass(e->Mfactor, solution, n);
        for (uint32_t r = 0; r < active; ++r) factor[r * stride + c] = solution[dofs[r]];
    }
    for (uint32_t r = 0; r < active; ++r)
        for (uint32_t c = 0; c < r; ++c) {
            const float v = 0.5f * (factor[r * stride + c] + factor[c * stride + r]);
            factor[r * stride + c] = factor[c * stride + r] = v;
        }
    if (!factor_control_mass(factor, active, stride, diagonal)) { e->status |= ORC_STATUS_CONTROL_FAILURE; return; }
    for (uint32_t c = 0; c < active; ++c) {
        for (uint32_t r = 0; r < active; ++r) rhs[r] = r == c ? 1.0f : 0.0f;
        solve_control_mass(factor, diagonal, active, stride, rhs, solution);
        for (uint32_t r = 0; r < active; ++r) mass[r * stride + c] = solution[r];
    }
    for (uint32_t r = 0; r < active; ++r) {
        double v = -m->damping[links[r]] * e->qdot[links[r]];
        for (uint32_t c = 0; c < active; ++c) v -= (double)mass[r * stride + c] * e->qddot[links[c]];
        bias[r] = (float)v;
    }
    if (m->cfg.control_mode == 4u) osc_command(m, e, active, links, dofs, mass, bias, stride);
    else {
        for (uint32_t c = 0; c < active; ++c) {
            const uint32_t l = links[c];
            rhs[c] = e->acc_target[l] + e->kp[l] * (e->drive_target[l] - e->q[l]) + e->kd[l] * (e->vel_target[l] - e->qdot[l]);
        }
        for (uint32_t r = 0; r < active; ++r) {
            double v = bias[r];
            for (uint32_t c = 0; c < active; ++c) v += (double)mass[r * stride + c] * rhs[c];
            e->drive_command[links[r]] = (float)v;
        }
    }
    for (uint32_t a = 0; a < active; ++a)
        if (!isfinite(e->drive_command[links[a]])) {
            for (uint32_t c = 0; c < active; ++c) e->drive_command[links[c]] = 0.0f;
            e->status |= ORC_STATUS_CONTROL_FAILURE;
            return;
        }
}

/* articulation.cu:259-277 JointTransform */
static void joint_transform(const orc_model *m, const orc_env *e, uint32_t l, float *X) {
    m3 jr = m3_ident();
    v3 tr = vadd(v3ld(m->local_pos + 3 * l), v3ld(m->parent_offset + 3 * l));
    if (m->jtype[l] == ORC_JOINT_REVOLUTE) jr = m3_axis_angle(v3ld(m->axis + 3 * l), e->q[l]);
    else if (m->jtype[l] == ORC_JOINT_PRISMATIC) {
        float rel[7]; joint_relative_frame(m, e, l, rel); tr = v3ld(rel);
    }
    m3 lr = m3_from_quat(qld(m->local_quat + 4 * l));
    make_motion_xf(m3_T(m3_mul(lr, jr)), tr, X);
}

/* articulation.cu:194-211 */
static void motion_subspace(uint32_t type, v3 axis, float *S) {
    z6(S);
    float ls = vdot(axis, axis);
    if (ls > 1.0e-12f) axis = vscale(axis, rsq(ls));
    if (type == ORC_JOINT_REVOLUTE) v3st(S, axis);
    else if (type == ORC_JOINT_PRISMATIC) v3st(S + 3, axis);
}

/* articulation.cu:309-376 PrepareArticulationKinematics (no external link wrench) */
static void prepare_kinematics(const orc_model *m, orc_env *e) {
    for (uint32_t l = 0; l < m->L; ++l) {
        if (m->parent[l] == ORC_NOLINK && m->jtype[l] == ORC_JOINT_FLOATING) {
            make_motion_xf(m3_ident(), V3(0, 0, 0), e->link_xup + 36 * l);
            z6(e->link_S + 6 * l);
            z6(e->link_vbias + 6 * l);
            continue;
        }
        joint_transform(m, e, l, e->link_xup + 36 * l);
        motion_subspace(m->jtype[l], v3ld(m->axis + 3 * l), e->link_S + 6 * l);
    }
    for (uint32_t l = 0; l < m->L; ++l) {
        const uint32_t p = m->parent[l];
        if (p == ORC_NOLINK && m->jtype[l] == ORC_JOINT_FLOATING) continue;
        float vp[6]; z6(vp);
        if (p != ORC_NOLINK) memcpy(vp, e->link_vel + 6 * p, 24);
        float tp[6], jv[6], v[6];
        xf_motion(e->link_xup + 36 * l, vp, tp);
        for (int i = 0; i < 6; ++i) jv[i] = e->link_S[6 * l + i] * e->qdot[l];
        for (int i = 0; i < 6; ++i) v[i] = tp[i] + jv[i];
        memcpy(e->link_vel + 6 * l, v, 24);
        motion_cross(v, jv, e->link_vbias + 6 * l);
    }
    for (uint32_t l = 0; l < m->L; ++l) {
        float iv[6];
        mat66_mulv(m->inertia + 36 * l, e->link_vel + 6 * l, iv);
        force_cross(e->link_vel + 6 * l, iv, e->link_pbias + 6 * l);
    }
}

/* articulation_mass.cuh:124-253 ComputeArticulationMass */
static void compute_mass(const orc_model *m, orc_env *e, const float *dissipation, float dt) {
    const uint32_t n = m->ndof, L = m->L;
    float *M = e->M;
    for (uint32_t i = 0; i < n * n; ++i) M[i] = 0.0f;
    memcpy(e->link_ic, m->inertia, sizeof(float) * 36 * L);
    for (uint32_t depth = m->max_depth; depth > 0u; --depth) {
        for (uint32_t l = 0; l < L; ++l) {
            if (m->depth[l] + 1u != depth) continue;
            for (uint32_t c = m->child_begin[l]; c < m->child_begin[l + 1]; ++c) {
                const uint32_t child = m->children[c];
                float d[36];
                xf_inertia_to_parent(e->link_xup + 36 * child, e->link_ic + 36 * child, d);
                for (int i = 0; i < 36; ++i) e->link_ic[36 * l + i] += d[i];
            }
        }
    }
    const int floating = L > 0 && m->parent[0] == ORC_NOLINK && m->jtype[0] == ORC_JOINT_FLOATING;
    if (floating && n >= 6u)
        for (uint32_t k = 0; k < 36u; ++k) M[(k / 6u) * n + k % 6u] = e->link_ic[k];
    for (uint32_t l = 0; l < L; ++l) {
        if (joint_dofs(m->jtype[l]) == 0u) continue;
        if (l == 0u && floating) continue;
        const uint32_t di = m->link_dof[l];
        if (di >= n) continue;
        float f[6];
        mat66_mulv(e->link_ic + 36 * l, e->link_S + 6 * l, f);
        float diag = dot6(e->link_S + 6 * l, f);
        diag += m->armature[l];
        if (dissipation) diag += dt * dissipation[l];
        M[di * n + di] = diag;
        uint32_t walk = l;
        for (;;) {
            const uint32_t p = m->parent[walk];
            if (p == ORC_NOLINK) break;
            float pushed[6];
            xf_force_T(e->link_xup + 36 * walk, f, pushed);
            memcpy(f, pushed, 24);
            walk = p;
            if (joint_dofs(m->jtype[walk]) == 0u) continue;
            const uint32_t dj = m->link_dof[walk];
            if (dj >= n) continue;
            if (walk == 0u && floating) {
                for (uint32_t b = 0; b < 6u && b < n; ++b) { M[di * n + b] = f[b]; M[b * n + di] = f[b]; }
                continue;
            }
            const float entry = dot6(e->link_S + 6 * walk, f);
            M[di * n + dj] = entry;
            M[dj * n + di] = entry;
        }
    }
}

/* articulation_mass.cuh:269-335 FactorMass: L D L^T, unit L below the diagonal, D on it. */
void orc_factor_mass(const float *M, float *F, uint32_t n) {
    float a[ORC_MAX_DOF][ORC_MAX_DOF];
    for (uint32_t i = 0; i < n; ++i) for (uint32_t j = 0; j <= i; ++j) a[i][j] = M[i * n + j];
    for (uint32_t i = 0; i < n * n; ++i) F[i] = 0.0f;
    for (uint32_t k = 0; k < n; ++k) {
        const float d = fmaxf(a[k][k], 1.0e-6f);
        F[k * n + k] = d;
        for (uint32_t i = k + 1; i < n; ++i) F[i * n + k] = a[i][k] / d;
        for (uint32_t i = k + 1; i < n; ++i) {
            const float l = F[i * n + k];
            for (uint32_t j = k + 1; j <= i; ++j) a[i][j] -= l * F[j * n + k] * d;
        }
    }
}

/* articulation_mass.cuh:357-411 SolveMassBlock / SolveMass */
void orc_solve_mass(const float *F, float *x, uint32_t n) {
    for (uint32_t j = 0; j < n; ++j)
        for (uint32_t i = j + 1; i < n; ++i) x[i] -= F[i * n + j] * x[j];
    for (uint32_t i = 0; i < n; ++i) x[i] /= F[i * n + i];
    for (uint32_t end = n; end > 0u; --end) {
        const uint32_t i = end - 1u;
        float s = x[i];
        for (uint32_t j = i + 1; j < n; ++j) s -= F[j * n + i] * x[j];
        x[i] = s;
    }
}

static float *dof_velocity(const orc_model *m, orc_env *e, uint32_t d, uint32_t *link, uint32_t *comp) {
    /* articulation_types.cuh:126-159 */
    for (uint32_t l = 0; l < m->L; ++l) {
        const uint32_t w = joint_dofs(m->jtype[l]);
        if (d < w) { *link = l; *comp = w == 1u ? ORC_NOLINK : d; return w == 1u ? &e->qdot[l] : &e->link_vel[6 * l + d]; }
        d -= w;
    }
    *link = ORC_NOLINK; *comp = ORC_NOLINK;
    return NULL;
}

/* articulation.cu:505-645 ArticulationDynamicsKernel with fold_drive_damping = 1 */
void orc_dynamics(const orc_model *m, orc_env *e, int integrate_velocity) {
    const uint32_t L = m->L, n = m->ndof;
    if (L == 0u) return;
    const v3 g = v3ld(m->cfg.gravity);
    const float dt = m->cfg.dt;
    prepare_kinematics(m, e);
    for (uint32_t l = 0; l < L; ++l) {
        float a[6];
        const uint32_t p = m->parent[l];
        if (p != ORC_NOLINK) xf_motion(e->link_xup + 36 * l, e->link_acc + 6 * p, a);
        else if (m->jtype[l] == ORC_JOINT_FLOATING) {
            v3 gl = qrot_inv(qld(e->base_pose + 3), g);
            z6(a); a[3] = -gl.x; a[4] = -gl.y; a[5] = -gl.z;
        } else {
            float world[6]; z6(world); world[3] = -g.x; world[4] = -g.y; world[5] = -g.z;
            xf_motion(e->link_xup + 36 * l, world, a);
        }
        for (int i = 0; i < 6; ++i) a[i] += e->link_vbias[6 * l + i];
        memcpy(e->link_acc + 6 * l, a, 24);
    }
    for (uint32_t l = 0; l < L; ++l) {
        float f[6];
        mat66_mulv(m->inertia + 36 * l, e->link_acc + 6 * l, f);
        for (int i = 0; i < 6; ++i) e->link_pbias[6 * l + i] += f[i];
    }
    for (uint32_t rem = m->max_depth + 1u; rem > 0u; --rem) {
        for (uint32_t l = 0; l < L; ++l) {
            if (m->depth[l] != rem - 1u) continue;
            for (uint32_t c = m->child_begin[l]; c < m->child_begin[l + 1]; ++c) {
                const uint32_t child = m->children[c];
                float f[6];
                xf_force_T(e->link_xup + 36 * child, e->link_pbias + 6 * child, f);
                for (int i = 0; i < 6; ++i) e->link_pbias[6 * l + i] += f[i];
            }
        }
    }
    float vel[ORC_MAX_DOF], acc[ORC_MAX_DOF];
    for (uint32_t d = 0; d < n; ++d) {
        uint32_t link, comp;
        float *v = dof_velocity(m, e, d, &link, &comp);
        const int scalar = comp == ORC_NOLINK;
        vel[d] = *v;
        e->bias[d] = scalar ? dot6(e->link_S + 6 * link, e->link_pbias + 6 * link) : e->link_pbias[6 * link + comp];
        const float damping = scalar ? m->damping[link] + e->drive_dissipation[link] : 0.0f;
        const float spring = scalar ? m->stiffness[link] * (e->q[link] - m->spring_ref[link]) : 0.0f;
        acc[d] = (scalar ? e->tau[link] : 0.0f) - e->bias[d] - damping * vel[d] - spring;
    }
    compute_mass(m, e, e->drive_dissipation, dt);
    orc_factor_mass(e->M, e->Mfactor, n);
    orc_solve_mass(e->Mfactor, acc, n);
    for (uint32_t l = 0; l < L; ++l) e->qddot[l] = 0.0f;
    for (uint32_t d = 0; d < n; ++d) {
        uint32_t link, comp;
        float *v = dof_velocity(m, e, d, &link, &comp);
        if (comp == ORC_NOLINK) {
            e->qddot[link] = acc[d];
            if (integrate_velocity) *v = vel[d] + dt * acc[d];
        } else if (integrate_velocity) {
            /* articulation.cu:603-615: the root's linear velocity steps with its origin's classical acceleration */
            const uint32_t i = comp % 3u, j = (i + 1u) % 3u, k = (i + 2u) % 3u;
            const float transport = comp < 3u ? 0.0f
                : vel[d - comp + j] * vel[d - i + k] - vel[d - comp + k] * vel[d - i + j];
            *v = vel[d] + dt * (acc[d] + transport);
        }
    }
    /* articulation.cu:617-644 final link accelerations */
    for (uint32_t l = 0; l < L; ++l) {
        float a[6];
        const uint32_t p = m->parent[l];
        if (m->jtype[l] == ORC_JOINT_FLOATING) {
            v3 gl = qrot_inv(qld(e->base_pose + 3), g);
            for (int c = 0; c < 6; ++c) a[c] = acc[c];
            a[3] -= gl.x; a[4] -= gl.y; a[5] -= gl.z;
        } else {
            if (p != ORC_NOLINK) xf_motion(e->link_xup + 36 * l, e->link_acc + 6 * p, a);
            else {
                float world[6]; z6(world); world[3] = -g.x; world[4] = -g.y; world[5] = -g.z;
                xf_motion(e->link_xup + 36 * l, world, a);
            }
            for (int c = 0; c < 6; ++c) a[c] += e->link_vbias[6 * l + c] + e->link_S[6 * l + c] * e->qddot[l];
        }
        memcpy(e->link_acc + 6 * l, a, 24);
    }
}

/* rigid_types.cuh:18-23 + symmetric_mat3 FromRotatedDiagonal: R diag(d) R^T */
static void world_inv_inertia(const float *pose, const float *iq, const float *inv_i, float *out) {
    quat q = qmul(qld(pose + 3), qld(iq));
    m3 R = m3_from_quat(q);
    float s[6] = {0, 0, 0, 0, 0, 0};
    const int ia[6] = {0, 1, 2, 0, 0, 1}, ib[6] = {0, 1, 2, 1, 2, 2};
    for (int k = 0; k < 6; ++k)
        for (int c = 0; c < 3; ++c) s[k] += R.m[ia[k] * 3 + c] * inv_i[c] * R.m[ib[k] * 3 + c];
    memcpy(out, s, 24);
}

/* articulation.cu:1019-1051 BodyIntegrateVelocityKernel (no external forces, no gravity compensation) */
void orc_body_integrate_velocity(const orc_model *m, orc_env *e) {
    const v3 g = v3ld(m->cfg.gravity);
    for (uint32_t b = 0; b < m->B; ++b) {
        if (m->inv_mass[b] <= 0.0f) { for (int k = 0; k < 6; ++k) e->body_winv[6 * b + k] = 0.0f; continue; }
        world_inv_inertia(e->body_pose + 7 * b, m->inertial_quat + 4 * b, m->inv_inertia + 3 * b, e->body_winv + 6 * b);
        if (m->body_to_link[b] != ORC_NOLINK) continue;   /* link mirrors carry no free dynamics */
        v3 v = v3ld(e->body_linvel + 3 * b);
        v3st(e->body_linvel + 3 * b, vadd(v, vscale(g, m->cfg.dt)));
    }
}

/* rigid_types.cuh:39-122 SolveFreeRotation */
static int solve_free_rotation(v3 w0, v3 inv_i, float dt, v3 *mid_out) {
    *mid_out = V3(0, 0, 0);
    v3 m0 = V3(w0.x / inv_i.x, w0.y / inv_i.y, w0.z / inv_i.z);
    float scale = fmaxf(fabsf(m0.x), fmaxf(fabsf(m0.y), fabsf(m0.z)));
    if (scale == 0.0f) return 0;
    v3 u0 = vscale(m0, 1.0f / scale);
    v3 a = vscale(inv_i, scale);
    v3 c = V3(dt * (a.y - a.z), dt * (a.z - a.x), dt * (a.x - a.y));
    v3 u = u0;
    float res = 0.0f;
    for (uint32_t it = 0; it <= 12u; ++it) {
        v3 mid = vscale(vadd(u0, u), 0.5f);
        v3 r = V3(u.x - u0.x + c.x * mid.y * mid.z, u.y - u0.y + c.y * mid.z * mid.x, u.z - u0.z + c.z * mid.x * mid.y);
        res = fmaxf(fabsf(r.x), fmaxf(fabsf(r.y), fabsf(r.z)));
        if (!isfinite(res)) return 1;
        if (res <= 1.0e-6f) { *mid_out = V3(a.x * mid.x, a.y * mid.y, a.z * mid.z); return 0; }
        if (it == 12u) break;
        float j[3][4] = {{1.0f, 0.5f * c.x * mid.z, 0.5f * c.x * mid.y, r.x},
                         {0.5f * c.y * mid.z, 1.0f, 0.5f * c.y * mid.x, r.y},
                         {0.5f * c.z * mid.y, 0.5f * c.z * mid.x, 1.0f, r.z}};
        for (int col = 0; col < 3; ++col) {
            int piv = col;
            for (int row = col + 1; row < 3; ++row) if (fabsf(j[row][col]) > fabsf(j[piv][col])) piv = row;
            if (!isfinite(j[piv][col]) || fabsf(j[piv][col]) < 1.0e-12f) return 1;
            for (int k = col; k < 4; ++k) { float t = j[col][k]; j[col][k] = j[piv][k]; j[piv][k] = t; }
            for (int row = col + 1; row < 3; ++row) {
                float f = j[row][col] / j[col][col];
                for (int k = col + 1; k < 4; ++k) j[row][k] -= f * j[col][k];
            }
        }
        v3 d;
        d.z = j[2][3] / j[2][2];
        d.y = (j[1][3] - j[1][2] * d.z) / j[1][1];
        d.x = (j[0][3] - j[0][1] * d.y - j[0][2] * d.z) / j[0][0];
        int accepted = 0; float alpha = 1.0f;
        for (int bt = 0; bt < 8; ++bt) {
            v3 t = vsub(u, vscale(d, alpha));
            v3 md = vscale(vadd(u0, t), 0.5f);
            v3 tr = V3(t.x - u0.x + c.x * md.y * md.z, t.y - u0.y + c.y * md.z * md.x, t.z - u0.z + c.z * md.x * md.y);
            float tres = fmaxf(fabsf(tr.x), fmaxf(fabsf(tr.y), fabsf(tr.z)));
            if (isfinite(tres) && tres < res) { u = t; accepted = 1; break; }
            alpha *= 0.5f;
        }
        if (!accepted) break;
    }
    return 1;
}

/* articulation.cu:732-791 IntegratePositionArticulationKernel + 1059-1116 BodyIntegratePositionKernel */
void orc_integrate_position(const orc_model *m, orc_env *e) {
    const float dt = m->cfg.dt;
    const int pseudo = m->cfg.pos_iters > 0u && e->row_cap > 0u;
    for (uint32_t l = 0; l < m->L; ++l) {
        const uint32_t d = m->link_dof[l];
        const int scalar = joint_dofs(m->jtype[l]) == 1u;
        if (pseudo && scalar) e->q[l] += (e->qdot[l] + e->qdot_pseudo[d]) * dt;
        else e->q[l] += e->qdot[l] * dt;
        if (m->parent[l] == ORC_NOLINK && m->jtype[l] == ORC_JOINT_FLOATING) {
            float *rv = e->link_vel + 6 * l, v[6];
            for (int i = 0; i < 6; ++i) v[i] = rv[i] + (pseudo ? e->qdot_pseudo[i] : 0.0f);
            quat rot = qld(e->base_pose + 3);
            v3 vw = qrot(rot, V3(v[3], v[4], v[5]));
            v3st(e->base_pose, vadd(v3ld(e->base_pose), vscale(vw, dt)));
            quat dq = Q4(1.0f, 0.5f * v[0] * dt, 0.5f * v[1] * dt, 0.5f * v[2] * dt);
            qst(e->base_pose + 3, qnorm_lt(qmul(rot, dq), 1.0e-24f));
            v3 turned = qrot_inv(qnorm_lt(dq, 1.0e-24f), V3(rv[3], rv[4], rv[5]));
            rv[3] = turned.x; rv[4] = turned.y; rv[5] = turned.z;
        }
    }
    /* the gyro bit is cleared before every body integration: ops/articulation.cu:1053-1056, 1810-1812 */
    if (m->B) e->status &= ~ORC_STATUS_GYRO_FAILURE;
    for (uint32_t b = 0; b < m->B; ++b) {
        if (m->inv_mass[b] <= 0.0f || m->body_to_link[b] != ORC_NOLINK) continue;
        float *pose = e->body_pose + 7 * b;
        v3 inv_i = v3ld(m->inv_inertia + 3 * b);
        quat principal = qnorm_le(qmul(qld(pose + 3), qld(m->inertial_quat + 4 * b)), 1.0e-12f);
        quat inverse = Q4(principal.w, -principal.x, -principal.y, -principal.z);
        v3 w0 = qrot(inverse, v3ld(e->body_angvel + 3 * b));
        v3 midpoint;
        if (solve_free_rotation(w0, inv_i, dt, &midpoint)) { e->status |= ORC_STATUS_GYRO_FAILURE; continue; }
        v3 momentum = qrot(principal, V3(w0.x / inv_i.x, w0.y / inv_i.y, w0.z / inv_i.z));
        v3 v = v3ld(e->body_linvel + 3 * b);
        v3 w = qrot(principal, midpoint);
        v3 center = vadd(v3ld(pose), qrot(qld(pose + 3), v3ld(m->inertial_pos + 3 * b)));
        quat dq = Q4(1.0f, 0.5f * dt * w.x, 0.5f * dt * w.y, 0.5f * dt * w.z);
        quat q = qnorm_le(qmul(dq, qld(pose + 3)), 1.0e-12f);
        if (pseudo) {
            v = vadd(v, v3ld(e->body_pseudo + 6 * b));
            v3 wp = v3ld(e->body_pseudo + 6 * b + 3);
            quat pq = Q4(1.0f, 0.5f * dt * wp.x, 0.5f * dt * wp.y, 0.5f * dt * wp.z);
            q = qnorm_le(qmul(pq, q), 1.0e-12f);
        }
        qst(pose + 3, q);
        v3 offset = qrot(q, v3ld(m->inertial_pos + 3 * b));
        v3st(pose, vsub(vadd(center, vscale(v, dt)), offset));
        world_inv_inertia(pose, m->inertial_quat + 4 * b, m->inv_inertia + 3 * b, e->body_winv + 6 * b);
        v3st(e->body_angvel + 3 * b, sym_mulv(e->body_winv + 6 * b, momentum));
    }
}

/* articulation.cu:647-689 FkLinkVelocitiesKernel */
void orc_fk_link_velocities(const orc_model *m, orc_env *e) {
    for (uint32_t l = 0; l < m->L; ++l) {
        const uint32_t p = m->parent[l];
        if (p == ORC_NOLINK && m->jtype[l] == ORC_JOINT_FLOATING) continue;
        float X[36], S[6], vp[6], v[6];
        joint_transform(m, e, l, X);
        motion_subspace(m->jtype[l], v3ld(m->axis + 3 * l), S);
        z6(vp);
        if (p != ORC_NOLINK) memcpy(vp, e->link_vel + 6 * p, 24);
        xf_motion(X, vp, v);
        for (int i = 0; i < 6; ++i) v[i] += S[i] * e->qdot[l];
        memcpy(e->link_vel + 6 * l, v, 24);
    }
}

/* articulation.cu:999-1016 ReadoutDrivesKernel: applied effort of each drive row */
void orc_readout_drives(const orc_model *m, orc_env *e) {
    for (uint32_t l = 0; l < m->L; ++l) e->actuator_applied[l] = 0.0f;
    for (uint32_t r = 0; r < e->nrows; ++r) {
        const orc_row *row = &e->rows[r];
        if (!(row->flags & ORC_ROW_ACTIVE) || row->tag != 3u) continue;
        const uint32_t l = row->link;
        e->actuator_applied[l] = row->lambda / m->cfg.dt - e->drive_dissipation[l] * e->qdot[l];
        e->tau[l] += e->actuator_applied[l];
    }
}
