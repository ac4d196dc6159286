// handles.hpp — definitions of the opaque host handles of the C ABI.
#pragma once
#include "../host/block_id.hpp"
#include "../host/page_pool.hpp"

struct nova_registry {
    novab::BlockRegistry r;
};
struct nova_pool {
    novab::PagePool p;
};
