// Pieces of the C-ABI translation unit shared with other files that export entry points.
#pragma once
#include <functional>

#include "../../include/b200idx.h"
#include "flat_index.h"

namespace b200_capi {
// Runs f, converts exceptions into status codes and records the message on the handle.
int guarded(const b200idx_t* h, const std::function<void()>& f);
// The exact-search object behind a Flat / Int8Flat handle, nullptr for other index types.
b200::FlatIndex* flat_of(b200idx_t* h);
}  // namespace b200_capi
