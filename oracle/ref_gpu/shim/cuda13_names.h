// Force-included ahead of the reference's CUDA sources: the reference is written against the CUDA 13 runtime, whose
// graph-capture entry points take edge data under their plain names; CUDA 12.9 spells those forms _v2 / _v3.  The
// overloads below forward the CUDA 13 argument lists to the 12.9 names.  Nothing else is changed.
#pragma once
#include <cuda_runtime.h>
static inline cudaError_t cudaGraphGetEdges(cudaGraph_t graph, cudaGraphNode_t* from, cudaGraphNode_t* to, cudaGraphEdgeData* edges, size_t* count) {
    return cudaGraphGetEdges_v2(graph, from, to, edges, count);
}
static inline cudaError_t cudaStreamGetCaptureInfo(cudaStream_t stream, cudaStreamCaptureStatus* status, unsigned long long* id, cudaGraph_t* graph,
                                                   const cudaGraphNode_t** deps, const cudaGraphEdgeData** edges, size_t* count) {
    return cudaStreamGetCaptureInfo_v3(stream, status, id, graph, deps, edges, count);
}
static inline cudaError_t cudaGraphAddNode(cudaGraphNode_t* node, cudaGraph_t graph, const cudaGraphNode_t* deps, const cudaGraphEdgeData* edges,
                                           size_t count, cudaGraphNodeParams* params) {
    return cudaGraphAddNode_v2(node, graph, deps, edges, count, params);
}
static inline cudaError_t cudaStreamUpdateCaptureDependencies(cudaStream_t stream, cudaGraphNode_t* deps, const cudaGraphEdgeData* edges, size_t count,
                                                              unsigned int flags) {
    return cudaStreamUpdateCaptureDependencies_v2(stream, deps, edges, count, flags);
}
