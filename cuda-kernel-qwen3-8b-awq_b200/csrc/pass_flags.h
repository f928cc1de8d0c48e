// Flags and tag constants of the operator-list pass kernel (decode_pass.cu), shared with the engine that builds its programs.
#pragma once

namespace qw3 {

constexpr int P_TAG_OPS = 1024;             // tags: launch epoch * P_TAG_OPS + operator index
constexpr int P_SRC_PEER = P_TAG_OPS - 1;   // `src` / `rsrc` of words the stage before this one stores from another GPU

enum PassOpFlags {
    PASS_WAIT_PREV = 1,   // inputs are plain memory written by the operator before: wait for its arrival counter
    PASS_PUBLISH = 2,     // the operator after (or the final arg-max) waits on this operator's arrival counter
    PASS_PEER_OUT = 4,    // yt is the next stage's inbox in another GPU's memory: system-scope stores, peer tag
    PASS_TOKEN_PEER = 8,  // embedding of a decode pass: the id arrives as a tagged word the last stage stores
};

}  // namespace qw3
