/*
 * Device wrapper of the deepRacin library, CUDA edition.  It keeps the function names
 * of the reference's OpenCL wrapper (include/dR_clwrap.h, src/dR_clwrap.c) so the graph
 * core and applications call the same entry points; each one now drives the CUDA
 * runtime: context = the device's primary context, command queue = a cudaStream_t,
 * cl_mem = a device pointer.  No kernel is compiled at run time: all kernels are built
 * for sm_100a ahead of time, so the source/program/kernel-object functions of the
 * reference have no counterpart.
 */
#ifndef DR_CLWRAP_H
#define DR_CLWRAP_H
#include "dR_base.h"
#ifdef __cplusplus
extern "C" {
#endif
/* Blocking host->device copy on the graph's stream; `offset` and `numBytes` in bytes
 * (reference src/dR_clwrap.c:1079-1143). */
gboolean dR_uploadArray(dR_Graph *net, gchar *name, void *srcHostMem, size_t offset, size_t numBytes, cl_mem destDeviceMem);
/* Blocking device->host copy; the only synchronisation point of an un-profiled run
 * (reference src/dR_clwrap.c:1145-1190). */
void dR_downloadArray(dR_Graph *net, gchar *name, cl_mem *srcDeviceMem, size_t byteOffset, size_t numBytes, void *destHostMem);
/* Allocates `size` floats of device memory (reference src/dR_clwrap.c:886-900). */
gboolean dR_createFloatBuffer(dR_Graph *net, cl_mem *mem, gint size, int buffertype);
/* Same for sizes beyond 2^31 floats-bytes products (batched activations). */
gboolean dR_createFloatBufferL(dR_Graph *net, cl_mem *mem, size_t numFloats);
/* Selects the device (clConfig->clDeviceNumber), retains its primary context and creates the
 * stream unless dR_setClEnvironment supplied one (reference dR_clInit, src/dR_clwrap.c:4-236). */
gboolean dR_clInit(dR_Graph *net);
/* With profilingGPU: closes the per-kernel event pair, prints the time and adds it to
 * totalKernelGPUTime; otherwise only checks for launch errors
 * (reference dR_finishCLKernel, src/dR_clwrap.c:955-1058). */
gboolean dR_finishCLKernel(dR_Graph *net, char *kernelName);
/* Starts the event pair dR_finishCLKernel closes. */
void dR_beginCLKernel(dR_Graph *net);
/* TRUE if clConfig->clError holds an error; prints it.  Unlike the reference
 * (src/dR_clwrap.c:874-883) it never tears the context down. */
gboolean dR_openCLError(dR_Graph *net, char *message, char *callerName);
gboolean dR_openCLErrorWithoutCleanup(dR_Graph *net, char *message, char *callerName);
gboolean dR_clMemoryBufferCleanup(dR_Graph *net, cl_mem mem);
gboolean dR_cleanupKernel(cl_kernel kernel);
gboolean dR_cleanupProgram(cl_program program);
/* Destroys the stream (if owned) and the profiling events (reference src/dR_clwrap.c:1193-1252). */
gboolean dR_cleanupCL(dR_Graph *net);
/* Downloads numFloats from deviceMem and writes them as one CSV line per 16 values
 * (reference src/dR_clwrap.c:1331-1407). */
gboolean dR_exportFloatArrayToCSV(dR_Graph *net, gchar *filepath, gchar *filename, cl_mem deviceMem, cl_float *hostMem, size_t numFloats);
/* Stream synchronise (clFinish). */
gboolean dR_finish(dR_Graph *net);
/* Pinned host memory helpers for overlapped feeds. */
void *dR_hostAllocPinned(size_t bytes);
void dR_hostFreePinned(void *p);
/* Non-blocking copies on the graph's stream (host memory should be pinned). */
gboolean dR_uploadArrayAsync(dR_Graph *net, void *srcHostMem, size_t numBytes, cl_mem destDeviceMem);
gboolean dR_downloadArrayAsync(dR_Graph *net, cl_mem srcDeviceMem, size_t numBytes, void *destHostMem);
/* Double-buffered feeding (see dR_setFeedOverlap): second stream + events, copy, and the two hooks dR_apply calls. */
gboolean dR_feedOverlapInit(dR_Graph *net, dR_Node *feed);
gboolean dR_feedOverlapCopy(dR_Graph *net, dR_Node *feed, void *srcHostMem, size_t numBytes);
gboolean dR_feedU8(dR_Graph *net, dR_Node *feed, const unsigned char *srcHostMem, size_t numBytes);
gboolean dR_feedOverlapBeforeApply(dR_Graph *net);
gboolean dR_feedOverlapAfterApply(dR_Graph *net);
void dR_feedOverlapCleanup(dR_Graph *net, dR_Node *feed);
/* device-side memset of floats to zero on the stream */
gboolean dR_zeroBuffer(dR_Graph *net, cl_mem mem, size_t numFloats);
/* Timing helpers for the autotuner: record start/stop on the stream, return elapsed ms. */
void dR_timerStart(dR_Graph *net);
gdouble dR_timerStopMs(dR_Graph *net);
/* CUDA-graph capture of a launch sequence on the graph's stream. */
gboolean dR_captureBegin(dR_Graph *net);
gboolean dR_captureEnd(dR_Graph *net);
gboolean dR_captureLaunch(dR_Graph *net);
void dR_captureDestroy(dR_Graph *net);
#ifdef __cplusplus
}
#endif
#endif
