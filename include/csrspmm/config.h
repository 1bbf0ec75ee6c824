// Compile-time constants shared by host and device code (reference: include/csrspmm/config.h:5).
#pragma once

namespace csrspmm {

static constexpr int WARP_SIZE = 32;

}
