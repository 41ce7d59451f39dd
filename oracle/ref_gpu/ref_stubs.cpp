// Test infrastructure.  The reference's .nks loader can follow references into MJCF / URDF / USD files; those
// importers need tinyxml2 and OpenUSD, which are absent on this machine, and no scene used here refers to such a
// file.  These definitions satisfy the linker and fail loudly if a scene ever reaches them.
#include <stdexcept>
#include <string>

#include "import/mjcf_importer.hpp"
#include "import/urdf_importer.hpp"
#include "import/usd_importer.hpp"

namespace nuka::import {
nuka::scene::SceneIR LoadMjcf(const std::string& path) { throw std::runtime_error("MJCF importer is not built here: " + path); }
nuka::scene::SceneIR LoadUrdf(const std::string& path, const UrdfImportOptions&) { throw std::runtime_error("URDF importer is not built here: " + path); }
nuka::scene::SceneIR LoadUsd(const std::string& path) { throw std::runtime_error("USD importer is not built here: " + path); }
bool IsUsdPath(const std::string&) { return false; }
}  // namespace nuka::import
