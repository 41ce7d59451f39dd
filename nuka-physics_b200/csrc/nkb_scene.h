// Scene cooking inside the library: `.nks` scene text in, cooked template bytes out (see nkb_scene.cpp).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "nkb_world.h"

namespace nkb {

constexpr uint32_t kEveryAdmissiblePair = 0xffffffffu;

struct CookOptions {
    float dt = 1.0f / 200.0f;
    uint32_t vel_iters = 4u, pos_iters = 32u;
    float kp = 0.0f, kd = 0.0f;            // drive gains of scalar joints that carry no actuator (0: undriven, as the reference cooks them)
    bool default_ground = false;           // add a plane at ground_height when the scene has no ground of its own
    float ground_height = 0.0f, ground_mu = 1.0f;
    bool self_collision = false;           // robot rows keep their own contype / conaffinity instead of "collides with the ground only"
    bool scene_filters = true;             // every row, the ground included, keeps the scene's contype / conaffinity bits
    // candidate-pair slots per env: 0 = one per shape row; kEveryAdmissiblePair = every pair the filters admit (the
    // reference's rule, src/scene/cook/cook_to_model.cpp:1541-1546), which the caller narrows after parsing
    uint32_t max_contacts = kEveryAdmissiblePair;
    uint32_t max_points = 0u;              // contact points per env with solver rows; 0 = derived bound, at most 128
};

// Cooks a scene document; throws Error (parse error, invalid argument, not supported) with a message.
std::vector<uint8_t> CookScene(const std::string& json_text, const CookOptions& options);

// CookScene, with kEveryAdmissiblePair resolved to the count of admissible pairs.
std::vector<uint8_t> CookSceneForWorld(const std::string& json_text, const CookOptions& options);

// True when the bytes start (after white space) like a JSON document rather than a cooked template.
bool LooksLikeScene(const std::string& bytes);

}  // namespace nkb
