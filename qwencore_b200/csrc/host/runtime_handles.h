// Opaque handle types behind the C API of the host runtime.
#pragma once

#include <memory>

#include "runtime.h"

// A cache handle either owns its CacheManager (qwc_cache_new) or views the one inside a
// scheduler (qwc_scheduler_cache).
struct qwc_cache {
    qwc::runtime::CacheManager* cache = nullptr;
    std::unique_ptr<qwc::runtime::CacheManager> owned;
};

struct qwc_scheduler {
    qwc::runtime::Scheduler scheduler;
    qwc_cache cache_view;
};
