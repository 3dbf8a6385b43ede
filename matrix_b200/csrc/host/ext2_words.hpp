// An extension-field element as the host layers pass it around: (c0, c1) words.
#pragma once
#include <cstdint>

namespace mbhost {

struct Ext2 {
    uint64_t c0 = 0, c1 = 0;
};

}  // namespace mbhost
