// One Net replica per GPU behind a single call: a host batch is cut into contiguous slices, every slice runs on its own
// GPU (own context, stream, caching allocator and weight replica) on its own host thread, and each slice's outputs land in
// the caller's buffers at the slice's offset. Images are independent and weights read-only, so there is no collective and
// no traffic between the GPUs; it replaces the reference's single entry Extractor::input / extract
// (Tensor/Net.cpp:686-736) for batches that one GPU should not run alone.
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/otter_b200_net.h"
#include "otter_api.hpp"

struct ott_net_group {
    std::vector<ott_net*> members;
    std::string error;
};

extern "C" {

void ott_net_group_partition(int n, int parts, int index, int* first, int* count) {
    // contiguous slices whose sizes differ by at most one image; the first n % parts slices take the extra image
    int f = 0, c = 0;
    if (parts > 0 && index >= 0 && index < parts && n > 0) {
        const int base = n / parts, extra = n % parts;
        f = index * base + (index < extra ? index : extra);
        c = base + (index < extra ? 1 : 0);
    }
    if (first) *first = f;
    if (count) *count = c;
}

int ott_net_group_create(const int* devices, int n_devices, ott_net_group** out) {
    if (!devices || n_devices < 1 || n_devices > 64 || !out) return OTT_ERR_INVALID;
    *out = nullptr;
    ott_net_group* g = new (std::nothrow) ott_net_group();
    if (!g) return OTT_ERR_ALLOC;
    for (int i = 0; i < n_devices; ++i) {
        ott_net* m = nullptr;
        const int rc = ott_net_create(devices[i], &m);
        if (rc != OTT_OK) {
            ott_net_group_destroy(g);
            return rc;
        }
        g->members.push_back(m);
    }
    *out = g;
    return OTT_OK;
}

int ott_net_group_destroy(ott_net_group* group) {
    if (!group) return OTT_OK;
    for (ott_net* m : group->members) ott_net_destroy(m);
    delete group;
    return OTT_OK;
}

int ott_net_group_size(const ott_net_group* group) { return group ? (int)group->members.size() : 0; }

ott_net* ott_net_group_member(ott_net_group* group, int index) {
    return (group && index >= 0 && index < (int)group->members.size()) ? group->members[(size_t)index] : nullptr;
}

const char* ott_net_group_last_error(const ott_net_group* group) { return group ? group->error.c_str() : "null group"; }

int ott_net_group_forward(ott_net_group* group, const char* input_blob, const float* in_host, int n, int c, int h, int w, int n_out,
                          const char* const* out_blobs, void* const* out_host) {
    if (!group || !input_blob || !in_host || n < 0 || n_out < 1 || !out_blobs || !out_host) return OTT_ERR_INVALID;
    const int parts = (int)group->members.size();
    group->error.clear();
    // bytes per image of every output blob in the layout ott_net_forward delivers (fp32 NCHW, or int8 NCHW for an int8 blob)
    std::vector<size_t> per_image((size_t)n_out);
    for (int i = 0; i < n_out; ++i) {
        int shape[4];
        if (!out_host[i]) { group->error = "ott_net_group_forward needs a host buffer for every output"; return OTT_ERR_INVALID; }
        if (ott_net_blob_shape(group->members[0], out_blobs[i], shape) != OTT_OK) { group->error = std::string("unknown blob ") + out_blobs[i]; return OTT_ERR_INVALID; }
        per_image[(size_t)i] = (size_t)shape[1] * shape[2] * shape[3] * (size_t)ott_net_blob_element_size(group->members[0], out_blobs[i]);
    }
    const size_t in_image = (size_t)c * h * w;
    std::vector<int> rcs((size_t)parts, OTT_OK);
    auto run = [&](int p) {
        int first = 0, count = 0;
        ott_net_group_partition(n, parts, p, &first, &count);
        if (count == 0) return;
        std::vector<void*> outs((size_t)n_out);
        for (int i = 0; i < n_out; ++i) outs[(size_t)i] = static_cast<char*>(out_host[i]) + per_image[(size_t)i] * (size_t)first;
        rcs[(size_t)p] = ott_net_forward(group->members[(size_t)p], input_blob, in_host + in_image * (size_t)first, 0, count, c, h, w, n_out, out_blobs,
                                         outs.data());
    };
    // one host thread per GPU (the calling thread takes the first slice): each enqueues and waits for its own device only
    std::vector<std::thread> workers;
    for (int p = 1; p < parts; ++p) workers.emplace_back(run, p);
    run(0);
    for (std::thread& t : workers) t.join();
    for (int p = 0; p < parts; ++p)
        if (rcs[(size_t)p] != OTT_OK) {
            group->error = "replica " + std::to_string(p) + ": " + ott_net_last_error(group->members[(size_t)p]);
            return rcs[(size_t)p];
        }
    return OTT_OK;
}

}  // extern "C"
