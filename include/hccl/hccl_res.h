/*
 * hccl_res.h -- the communicator-side resources an operator developer builds on.
 *
 * In HCCL these calls come from the separate communication base library (reference declarations:
 * src/common/hcomm_dlsym/hccl_host_comm_dl.h:43-58, hccl_res_dl.h:73-118, hccl_rank_graph_dl.h:38-49,
 * hccl_res_expt_dl.h:25-27); here they are part of the same library. "Threads", "channels" and "notifies" have no
 * counterpart objects: a thread is a CUDA stream, a channel is a peer mapping of the symmetric heap, a notify is a
 * flag word in it (hccl_comm.h: HcclCommSymAlloc / HcclSymWinGetPeerPointer / HcclSymGetMulticastPointer).
 */
#ifndef HCCL_B200_RES_H_
#define HCCL_B200_RES_H_

#include "hccl_comm.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- communicator state ------------------------------------------------------------------------------------------ */
typedef void (*HcclCommStateCallback)(void *userData, HcclCommStatus newStatus);
/* Called (from the thread that detects it: an API call, or the heartbeat watchdog) whenever the communicator turns
 * SUSPENDING or READY again. */
HcclResult HcclCommRegCommStateCallback(HcclComm comm, HcclCommStateCallback cb, void *userData);
/* The configuration the communicator was created with, defaults filled in. */
HcclResult HcclConfigGetInfo(HcclComm comm, HcclCommConfig *config);
/* Status of the communicator of this process that carries `group` as its name. */
HcclResult HcclGroupStatusGet(const char *group, HcclCommStatus *status);

/* ---- keyed blobs attached to a communicator (caches of an operator: topology digests, plans, kernel arguments) ---- */
typedef enum { HCCL_CTX_HOST = 0, HCCL_CTX_DEVICE = 1 } HcclCtxPlace;
HcclResult HcclEngineCtxCreate(HcclComm comm, const char *tag, HcclCtxPlace place, uint64_t size, void **ptr);
HcclResult HcclEngineCtxGet(HcclComm comm, const char *tag, HcclCtxPlace place, void **ptr, uint64_t *size);   /* HCCL_E_NOT_FOUND if absent */
HcclResult HcclEngineCtxCopy(HcclComm comm, const char *tag, const void *hostSrc, uint64_t size);             /* host -> blob */
HcclResult HcclEngineCtxDestroy(HcclComm comm, const char *tag);

/* ---- memory registration ------------------------------------------------------------------------------------------
 * Memory that peers may address must live in the symmetric heap: HcclCommMemReg accepts a range inside an
 * HcclCommSymAlloc allocation (or the CCL buffer) and returns its window offset, identical on every rank; any other
 * pointer is refused with HCCL_E_NOT_SUPPORT (copy through the CCL buffer instead, as the operators do). */
HcclResult HcclCommMemReg(HcclComm comm, void *addr, uint64_t size, uint64_t *windowOffset);
HcclResult HcclCommMemDereg(HcclComm comm, void *addr);

/* HcclMemAlloc = HcclCommSymAlloc + HcclCommMemReg of the whole block; HcclMemFree drops the window and returns the block.
 * Collective in the same sense as HcclCommSymAlloc: every rank issues the same sequence of calls (no communication happens).
 *
 * Allocator hooks for frameworks that take a pair of C functions (e.g. torch.cuda.memory.CUDAPluggableAllocator):
 * HcclSetAllocatorComm names the communicator whose heap serves the hooks (NULL detaches; destroying that communicator
 * detaches too); HcclAllocHook returns NULL when no communicator is attached, it lives on another device, or its heap is
 * full; HcclFreeHook ignores pointers whose communicator is gone (the heap went with it). */
HcclResult HcclMemAlloc(HcclComm comm, uint64_t bytes, void **ptr);
HcclResult HcclMemFree(HcclComm comm, void *ptr);
HcclResult HcclSetAllocatorComm(HcclComm comm);
HcclResult HcclGetAllocatorComm(HcclComm *comm);          /* NULL when nothing (live) is attached */
void *HcclAllocHook(long long bytes, int device, void *stream);
void HcclFreeHook(void *ptr, long long bytes, int device, void *stream);

/* ---- rank graph (topology as layers of fully connected groups) ---------------------------------------------------- */
typedef enum { HCCL_TOPO_CLOS = 0, HCCL_TOPO_MESH_1D = 1, HCCL_TOPO_MESH_1D_CLOS = 2, HCCL_TOPO_NVSWITCH = 3 } HcclTopoType;
typedef enum { HCCL_LINK_NONE = 0, HCCL_LINK_NVLINK = 1, HCCL_LINK_PCIE = 2, HCCL_LINK_SHM = 3, HCCL_LINK_NET = 4 } HcclLinkType;
typedef struct HcclLinkInfoDef {
    HcclLinkType type;
    uint32_t layer;               /* lowest layer at which the two ranks share a group */
    double bandwidthGBs;          /* per direction */
    uint32_t peerAccess;          /* 1: loads / stores reach the peer's heap directly */
} HcclLinkInfo;
HcclResult HcclRankGraphGetLayers(HcclComm comm, uint32_t *numLayers);
/* Ranks of the group this rank belongs to at `layer`; *num is capacity on entry, count on return. */
HcclResult HcclRankGraphGetRanksByLayer(HcclComm comm, uint32_t layer, uint32_t *ranks, uint32_t *num);
/* Sizes of all groups ("topology instances") of a layer. */
HcclResult HcclRankGraphGetInstSizeListByLayer(HcclComm comm, uint32_t layer, uint32_t *sizes, uint32_t *num);
HcclResult HcclRankGraphGetTopoTypeByLayer(HcclComm comm, uint32_t layer, HcclTopoType *type);
HcclResult HcclRankGraphGetLinks(HcclComm comm, uint32_t srcRank, uint32_t dstRank, HcclLinkInfo *link);

/* ---- small blobs published to the other ranks (what HCCL piggy-backs on channel setup) ----------------------------- */
HcclResult HcclCommAddExchangeInfo(HcclComm comm, const char *key, const void *data, uint32_t size);
/* Blocks (up to the connect timeout) until `rank` has published `key`. *size is capacity on entry, length on return. */
HcclResult HcclCommGetExchangeInfo(HcclComm comm, uint32_t rank, const char *key, void *data, uint32_t *size);

#ifdef __cplusplus
}
#endif
#endif
