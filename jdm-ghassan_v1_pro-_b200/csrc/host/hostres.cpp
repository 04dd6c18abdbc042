#include "hostres.hpp"

#include <sys/stat.h>
#include <sys/statvfs.h>
#include <unistd.h>

#include <algorithm>
#include <filesystem>
#include <set>
#include <utility>

namespace fs = std::filesystem;

namespace gbh {

uint64_t physical_ram_bytes() {
  const long pages = sysconf(_SC_PHYS_PAGES), page = sysconf(_SC_PAGE_SIZE);
  if (pages <= 0 || page <= 0) return 0;
  return static_cast<uint64_t>(pages) * static_cast<uint64_t>(page);
}

uint64_t free_disk_bytes(const std::string& path) {
  std::error_code ec;
  fs::path p = fs::absolute(fs::path(path.empty() ? "." : path), ec);
  if (ec) return 0;
  // walk up to something that exists: the checkpoint directory is usually created later
  for (int i = 0; i < 64 && !p.empty(); ++i) {
    if (fs::exists(p, ec) && !ec) break;
    if (!p.has_parent_path() || p.parent_path() == p) break;
    p = p.parent_path();
  }
  struct statvfs sv;
  if (statvfs(p.c_str(), &sv) != 0) return 0;
  return static_cast<uint64_t>(sv.f_bavail) * static_cast<uint64_t>(sv.f_frsize);
}

TreeSize tree_size_bytes(const std::string& root, const std::vector<std::string>& skip_dirs) {
  TreeSize out;
  std::error_code ec;
  if (!fs::is_directory(root, ec) || ec) return out;
  std::set<std::pair<uint64_t, uint64_t>> seen;   // (device, inode)
  std::vector<fs::path> stack{fs::path(root)};
  while (!stack.empty()) {
    const fs::path dir = stack.back();
    stack.pop_back();
    fs::directory_iterator it(dir, fs::directory_options::skip_permission_denied, ec), end;
    if (ec) { ec.clear(); continue; }
    for (; it != end; it.increment(ec)) {
      if (ec) { ec.clear(); break; }
      struct stat st;
      if (lstat(it->path().c_str(), &st) != 0) continue;
      if (S_ISDIR(st.st_mode)) {
        const std::string name = it->path().filename().string();
        if (std::find(skip_dirs.begin(), skip_dirs.end(), name) == skip_dirs.end()) stack.push_back(it->path());
      } else if (S_ISREG(st.st_mode)) {
        if (seen.emplace(static_cast<uint64_t>(st.st_dev), static_cast<uint64_t>(st.st_ino)).second) {
          out.bytes += static_cast<uint64_t>(st.st_size);
          out.unique_files += 1;
        }
      }
    }
  }
  return out;
}

}  // namespace gbh
