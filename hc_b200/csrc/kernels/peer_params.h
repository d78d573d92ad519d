// Destinations of a kernel that writes its result into several buffers at once:
// its own GPU's copy of the full output and the copies of the other GPUs of a
// multi-GPU job (peer memory reached over NVLink).  Shared by the kernels and by
// the host code that fills it.
#pragma once

constexpr int HC_MAX_PEERS = 8;

struct HcPeerDsts {
  void *base[HC_MAX_PEERS]; // this kernel's row 0 in every destination
  int count;                // 1..HC_MAX_PEERS
};
