/*
 * Graph, node and configuration types of the deepRacin C API, re-declared for the
 * CUDA (sm_100a) build.  Struct, field, enum and typedef names follow the
 * reference's include/dR_types.h:17-228 because applications reach into them
 * directly (examples/vgg16/vgg_deployed.c:108-116 sets net->config->... and
 * net->clConfig->clPlatformName).  The OpenCL handle types are mapped onto CUDA:
 *
 *   cl_mem            device pointer (float data)
 *   cl_command_queue  cudaStream_t
 *   cl_context        CUcontext of the device's primary context (informational)
 *   cl_device_id      device ordinal
 *   cl_platform_id    unused
 *   cl_kernel         unused (kernels are precompiled; a node records its variant instead)
 *
 * Fields after the "b200" markers are additions of this build.
 */
#ifndef DR_TYPES_H
#define DR_TYPES_H
#include "dR_compat.h"

typedef void *cl_mem;
typedef void *cl_command_queue;
typedef void *cl_context;
typedef void *cl_platform_id;
typedef intptr_t cl_device_id;
typedef void *cl_kernel;
typedef void *cl_program;
typedef void *cl_event;
typedef float cl_float;
typedef int cl_int;
typedef unsigned int cl_uint;
typedef unsigned long cl_ulong;
typedef int cl_build_status;
#define CL_MEM_READ_WRITE 1
#define CL_MEM_READ_ONLY 4
#define CL_DEVICE_TYPE_GPU (1 << 2)

typedef struct dR_Config dR_Config;
typedef struct dR_ClConfig dR_ClConfig;
typedef struct dR_Node dR_Node;
typedef struct dR_Graph dR_Graph;
typedef struct dR_ListElement dR_ListElement;
typedef struct dR_List dR_List;
typedef struct dR_DataFeedNode_Data dR_DataFeedNode_Data;
typedef struct dR_MemoryHandler dR_MemoryHandler;
typedef struct dR_Shape2 dR_Shape2;
typedef struct dR_Shape3 dR_Shape3;
typedef struct dR_Shape4 dR_Shape4;

/* Per-node function slots (reference include/dR_types.h:32-48). */
typedef gboolean (*fCompute)(dR_Graph *net, dR_Node *layer);
typedef gboolean (*fSchedule)(dR_Graph *net, dR_Node *layer);
typedef gboolean (*fPropagate)(dR_Graph *net, dR_Node *layer);
typedef gint32 (*fMaxBuffer)(dR_Node *layer);
typedef gboolean (*fCreateKernel)(dR_Graph *net, dR_Node *layer);
typedef gboolean (*fAllocateBuffers)(dR_Graph *net, dR_Node *layer);
typedef gboolean (*fFillBuffers)(dR_Graph *net, dR_Node *layer);
typedef gboolean (*fCleanupBuffers)(dR_Graph *net, dR_Node *layer);
typedef gboolean (*fCleanupLayer)(dR_Graph *net, dR_Node *layer);
typedef gchar *(*fPrintLayer)(dR_Node *layer);
typedef gchar *(*fSerializeNode)(dR_Node *layer, gchar *params[], gint *numParams, gfloat *variables[],
                                 gint variableSizes[], gint *numVariables);
typedef dR_Node *(*fParseAppendNode)(dR_Graph *net, dR_Node **iNodes, gint numINodes, gchar **params,
                                     gint numParams, gfloat **variables, gint numVariables);
typedef gboolean (*fGenerateKernel)(dR_Graph *net, dR_Node *layer);
typedef gchar *(*fCreateKernelName)(dR_Node *layer);
typedef void (*fSetVariables)(dR_Node *layer, gfloat *weights, gfloat *bias);

struct dR_Shape2 { gint s0; gint s1; };
struct dR_Shape3 { gint s0; gint s1; gint s2; };           /* (W, H, C) for tensors */
struct dR_Shape4 { gint s0; gint s1; gint s2; gint s3; };

enum dR_LayerType {
    tPooling, tBN, tFullyConnected, tConv2d, tPPFilter, tMaskDependentFilter, tLabelCreation,
    tNormalization, tUpscaling, tRGB2Gray, tMulScalar, tAddScalar, tDataFeedNode, tResolveRoI,
    tSoftmax, tSlice, tConcat, tCropOrPad, tElemWise2Op, tElemWise1Op, tFFT
};
typedef enum dR_LayerType dR_LayerType;

enum dR_ActivationType { tLinear, tReLU, tSigmoid /* unsupported */, tTan /* unsupported */ };
typedef enum dR_ActivationType dR_ActivationType;

struct dR_DataFeedNode_Data {
    dR_Shape3 shape;
    cl_mem dataBuffer;
    dR_List *next_layers;
    /* ---- b200 additions: double-buffered feeding (dR_setFeedOverlap) ---- */
    cl_mem feedBuf[2];       /* the two interface buffers the copy stream alternates between */
    void *evReady[2];        /* copy into feedBuf[i] finished (recorded on the copy stream) */
    void *evFree[2];         /* the apply that read feedBuf[i] finished (recorded on the compute stream) */
    gint current;            /* buffer the graph reads in the next apply */
    gint pending;            /* buffer a dR_feedDataAsync filled since the last apply, or -1 */
    cl_mem u8Buf[2];         /* device staging for 8-bit feeds (dR_feedDataU8Async), allocated at the first such feed */
};

struct dR_Node {
    dR_Shape3 oshape;
    gint32 layerID;
    dR_List *previous_layers;
    dR_List *next_layers;
    cl_kernel clKernel;
    dR_MemoryHandler *outputBuf;   /* the buffer the API hands out for this node (interface layout) */
    void *layer;
    dR_LayerType type;
    gboolean propagated;
    gboolean output;
    gboolean queued;

    fCompute compute;
    fSchedule schedule;
    fPropagate propagateShape;
    fMaxBuffer getRequiredOutputBufferSize;
    fCreateKernel createKernel;
    fAllocateBuffers allocateBuffers;
    fFillBuffers fillBuffers;
    fCleanupBuffers cleanupBuffers;
    fCleanupLayer cleanupLayer;
    fPrintLayer printLayer;
    fSerializeNode serializeNode;
    fParseAppendNode parseAppendNode;

    fGenerateKernel generateKernel;
    fCreateKernelName createKernelName;
    fSetVariables setVariables;

    /* ---- b200 additions ---- */
    dR_MemoryHandler *act;   /* activations in the internal N-HWC layout (== outputBuf when the two
                                layouts coincide and the node is neither feed nor output) */
    gint act_cstride;        /* channel stride (floats per pixel) of `act`; > oshape.s2 when the node
                                writes straight into a Concat consumer's buffer */
    gint act_coffset;        /* channel offset inside that pixel */
    gboolean elided;         /* node produces its result in place of a consumer's buffer / is skipped */
    gboolean fusedAway;      /* a consumer evaluates this node as part of its own kernel: compute() is not called */
    size_t scratchFloats;    /* per-apply scratch this node needs (shared, graph-owned) */
    gdouble lastGpuMs;       /* per-node kernel time of the last profiled apply */
};

struct dR_ClConfig {
    cl_context clContext;
    cl_platform_id clPlatformId;
    cl_command_queue clCommandQueue;   /* cudaStream_t all kernels and copies are issued on */
    cl_program clProgram;
    cl_uint clDeviceType;
    cl_uint clDeviceNumber;            /* CUDA device ordinal chosen by dR_initCL */
    gchar *clPlatformName;
    gchar *clKernelPath;
    cl_device_id clDeviceId;
    cl_uint clNumDevices;
    cl_device_id clDeviceIds[20];
    gchar *clDeviceName;
    cl_int clError;                    /* last cudaError_t */
    cl_event clEventObject;
    cl_event *clEvent;
    gboolean forceRecompile;
    gdouble totalKernelGPUTime;
    gdouble queueKernelGPUTime;
    gdouble maxTotalKernelGPUTime;
    gdouble sumTotalKernelGPUTime;
    gboolean clInfo;
    gboolean fastRelaxedMath;
    cl_build_status build_status;
    gboolean cleanupDone;
    gchar *configH;
    glong memConsumptionGPU;
    /* ---- b200 additions ---- */
    gboolean ownsStream;               /* stream was created by dR_initCL (destroyed at cleanup) */
    void *evStart, *evStop;            /* cudaEvent_t pair for per-node profiling */
    void *copyStream;                  /* second stream for overlapped feeds */
    gint smCount;
    size_t smemPerBlockOptin;
    void *uploadStage;                 /* pinned staging buffer of the blocking upload (pageable sources), allocated at the first large upload */
    size_t uploadStageBytes;
};

struct dR_Config {
    gboolean silent;
    gboolean profilingGPU;
    gboolean profilingCPU;
    gboolean debugInfo;
    gdouble totalNodeCPUTime;
    gint convLocalWorkSizeWindow;
    gchar *modelPath;
    /* ---- b200 additions ---- */
    gint batchSize;          /* images per dR_apply (the reference has none: one image per apply) */
    gint mathMode;           /* dR_MathMode */
    gint interfaceLayout;    /* dR_InterfaceLayout of feed / output buffers */
    gint convAlgo;           /* graph-wide dR_ConvAlgo override (DR_CONV_AUTO = per node) */
    gboolean autotune;       /* time the legal conv variants per layer during dR_prepare */
    gboolean fuseGraph;      /* enable concat elision / preamble folding */
    gboolean useCudaGraph;   /* replay the node schedule from a captured CUDA graph */
    gboolean feedOverlap;    /* dR_feedDataAsync copies on a second stream into alternating buffers */
    gboolean dryRun;         /* plan only: no device is touched, buffers get placeholder addresses, dR_apply refuses */
    size_t dryRunCursor;
};

struct dR_Graph {
    gboolean prepared;
    cl_mem swapBuffer1;
    cl_mem swapBuffer2;
    dR_Config *config;
    dR_ClConfig *clConfig;
    dR_List *feed_layers;
    dR_List *output_layers;
    dR_List *streamBufferHandlers;
    gint32 number_of_layers;
    gint32 maxBufferSize;
    cl_float *hostDebugBuffer;
    dR_List *scheduledLayers;
    dR_List *allNodes;
    gint debugLayer;
    /* ---- b200 additions ---- */
    cl_mem scratch;          /* shared per-apply scratch (Winograd transform domain, FC partials) */
    size_t scratchFloats;
    void *graphExec;         /* cudaGraphExec_t when useCudaGraph */
    size_t captureKey;       /* hash of the feed / output buffer addresses the captured graph was recorded with */
    gint deviceStatus;       /* last non-zero status a kernel reported (bounded waits etc.) */
    cl_mem statusWord;       /* device int the tensor-core kernels write error codes to */
};

struct dR_MemoryHandler {
    dR_List *outputFor;
    gint size;                         /* floats per image */
    gint numberOfDependencies;
    cl_mem *bufptr;
    cl_mem buf;
    gboolean outputBuf;                /* user supplied: never allocated or freed by the graph */
    gboolean regionOfInterest;
    gboolean useIndexBufferForRoI;
    cl_mem *indexBuffer;
    gint index;
    dR_Shape3 roiOrigin;
};

struct dR_ListElement {
    dR_ListElement *next;
    dR_ListElement *previous;
    void *element;
};

struct dR_List {
    dR_ListElement *first;
    dR_ListElement *last;
    gint length;
    dR_ListElement *iterator;
};

#define DEVICE_TYPE_DEFAULT (1 << 0)
#define DEVICE_TYPE_CPU (1 << 1)
#define DEVICE_TYPE_GPU (1 << 2)
#define DEVICE_TYPE_ACCELERATOR (1 << 3)
#define DEVICE_TYPE_ALL 0xFFFFFFFF

#endif /* DR_TYPES_H */
