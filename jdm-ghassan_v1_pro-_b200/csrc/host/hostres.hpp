// Host resources the trainer checks before it starts (the reference's core/device.cpp:65-354 has the same three
// probes): physical RAM, free bytes on the volume of a path, and the bytes below a directory with every hard-linked
// file counted once (best.ckpt and last.ckpt are often one file with two names).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace gbh {

uint64_t physical_ram_bytes();
// Free bytes available to this user on the volume that holds `path` (or its nearest existing parent); 0 = unknown.
uint64_t free_disk_bytes(const std::string& path);
struct TreeSize {
  uint64_t bytes = 0;
  uint64_t unique_files = 0;
};
// Regular files below `root`, each inode once; directories whose base name is in `skip_dirs` are not entered and
// symbolic links are not followed.  A missing root gives zeros.
TreeSize tree_size_bytes(const std::string& root, const std::vector<std::string>& skip_dirs);

}  // namespace gbh
