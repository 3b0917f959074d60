// Peer-visible memory shared by the collective kernels (q4_comm.cu) and the fused decode kernel (q4_fused.cu).
#pragma once
#include "q4_common.cuh"

constexpr int kLLMaxDim = 16384;        // largest model dimension the tagged residual-stream exchange holds
constexpr int kLLMaxVocab = 256 * 1024; // largest vocabulary of the gathered logits

// Tagged ("LL") exchange area of one rank, written by every rank (itself included) with plain peer stores:
//   x[b][r][n]   partial of residual-stream element n from source rank r, buffer b (the two all-reduces of a layer
//                alternate buffers); a 32-bit word = fp16 value | tag << 16, so readers poll the data itself
//   cand[b][r]   rank r's argmax candidate (two tagged 64-bit words: value bits, global index), b = token parity
//   logits       all ranks' logits slices (plain fp16), complete once every candidate has arrived
struct Q4LLArea {
    uint32_t x[2][Q4_MAX_GPUS][kLLMaxDim];
    unsigned long long cand[2][Q4_MAX_GPUS][2];
    uint16_t logits[kLLMaxVocab];
};

int q4_comm_world(const q4_comm* c);
int q4_comm_rank(const q4_comm* c);
// LL area of rank `peer`, as a pointer that is valid on the calling rank's device.
Q4LLArea* q4_comm_ll_area(const q4_comm* c, int peer);
// True when a message of `count` halfs goes through NCCL on this communicator (backend choice, NCCL attached).
bool q4_comm_prefers_nccl(const q4_comm* c, int count);
// The in-place sum all-reduce through the peer-push kernel whatever the backend setting (count <= Q4_COMM_MAX_HALFS).
int q4_all_reduce_peer_push(q4_comm* c, void* stream, uint16_t* buf, int count);
