// Minimal stand-in for faiss::ClusteringParameters (NOT Faiss): field order and defaults follow
// the published struct so that configs embedding it keep their layout.
#pragma once
namespace faiss {
struct ClusteringParameters {
    int niter = 25;
    int nredo = 1;
    bool verbose = false;
    bool spherical = false;
    bool int_centroids = false;
    bool update_index = false;
    bool frozen_centroids = false;
    int min_points_per_centroid = 39;
    int max_points_per_centroid = 256;
    int seed = 1234;
    size_t decode_block_size = 32768;
};
}  // namespace faiss
