// Peer-to-peer (NVLink / NVSwitch) kernels: see p2p.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
