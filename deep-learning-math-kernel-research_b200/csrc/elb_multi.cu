// Two callers' conveniences on top of the per-layer plans (include/euler_b200.h):
//
//   elb_stack_*        a chain of convolutions that stays on the device: layer k's output tensor is
//                      layer k+1's input (u8 between int8 layers, fp32 between fp32 layers), with an
//                      optional spatial subsample behind a layer.  The reference's harness runs
//                      chains this way on the host (tests/elt_conv.cpp:399-410, the --output_as_input
//                      and --dbuffering modes); here the whole chain is one call and, for host
//                      tensors, one CUDA graph per staging slot.
//   elb_conv_multi_*   one convolution whose minibatch is split over several GPUs of one box: GPU r
//                      runs images [r*N/G, (r+1)*N/G) with its own copy of the prepared weights, no
//                      exchange step.  The reference partitions the same loop (images / tiles
//                      outermost) over OpenMP threads (src/elx_conv_wino_xopt.hpp:41-64,
//                      src/elx_int8_conv_direct_1x1_xopt.hpp:91-97).
//
// Both are plain host code over the C-ABI entry points of elb_api.cu; no kernel lives here.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/euler_b200.h"

namespace elb {
void set_last_error(const char *msg);   // elb_api.cu
}

namespace {

int mfail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  elb::set_last_error(buf);
  return code;
}

#define M_TRY(expr)                                                                               \
  do {                                                                                            \
    cudaError_t e__ = (expr);                                                                     \
    if (e__ != cudaSuccess)                                                                       \
      return mfail(ELB_GENERAL_ERROR, "CUDA error %s at %s:%d (%s)", cudaGetErrorName(e__), __FILE__, __LINE__, \
                   cudaGetErrorString(e__));                                                      \
  } while (0)

struct DevGuard {
  int prev = -1;
  explicit DevGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DevGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

bool on_device(const void *p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

size_t elem_bytes(int dt) { return dt == ELB_F32 ? 4 : dt == ELB_F16 ? 2 : 1; }

}  // namespace

// ================================================================================== stack
struct elb_stack {
  struct Layer {
    elb_conv_t *plan = nullptr;
    elb_conv_desc_t d{};
    elb_conv_info_t info{};
    int step = 1;               // subsample behind this layer (1 = none)
    bool fused = false;         // ... which the NEXT layer folds into its input loads (no kernel, no d_sub)
    void *d_out = nullptr;      // this layer's output (null for the last layer without a subsample: the caller's tensor)
    void *d_sub = nullptr;      // the subsampled tensor (null when step == 1, or when it is the caller's tensor)
    bool prepared = false;
  };
  std::vector<Layer> layers;
  int device = 0, n = 0;
  size_t in_bytes = 0, out_bytes = 0;     // one batch of n images, caller's side
  uint64_t extra_launches = 0;            // subsample kernels
  std::vector<cudaEvent_t> layer_ev;      // optional: recorded before every layer and after the last one
  // host-tensor execution: two staging slots, a graph of the chain per slot
  cudaStream_t s_run = nullptr, s_h2d = nullptr, s_d2h = nullptr;
  void *stage_in[2] = {nullptr, nullptr}, *stage_out[2] = {nullptr, nullptr};
  cudaGraphExec_t graph[2] = {nullptr, nullptr};
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_run[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  // kernel launches: the plans count what was enqueued; enqueues made while capturing launched
  // nothing (capture_counted), every replay of a slot's graph launches one chain
  uint64_t graph_replays = 0, launches_per_chain = 0, capture_counted = 0;

  ~elb_stack() {
    DevGuard g(device);
    for (cudaStream_t s : {s_run, s_h2d, s_d2h}) if (s) { cudaStreamSynchronize(s); }
    for (int i = 0; i < 2; ++i) {
      if (graph[i]) cudaGraphExecDestroy(graph[i]);
      for (cudaEvent_t e : {ev_in[i], ev_run[i], ev_out[i]}) if (e) cudaEventDestroy(e);
      if (stage_in[i]) cudaFree(stage_in[i]);
      if (stage_out[i]) cudaFree(stage_out[i]);
    }
    for (cudaStream_t s : {s_run, s_h2d, s_d2h}) if (s) cudaStreamDestroy(s);
    for (Layer &l : layers) {
      if (l.d_out) cudaFree(l.d_out);
      if (l.d_sub) cudaFree(l.d_sub);
      if (l.plan) elb_conv_destroy(l.plan);
    }
  }
};

namespace {

// Enqueue the whole chain for one batch on stream s (device pointers).
int stack_enqueue(elb_stack &st, void *output, const void *input, cudaStream_t s) {
  const void *x = input;
  const size_t L = st.layers.size();
  for (size_t k = 0; k < L; ++k) {
    elb_stack::Layer &l = st.layers[k];
    const bool last = k + 1 == L;
    void *y = (last && l.step == 1) ? output : l.d_out;
    if (!st.layer_ev.empty() && cudaEventRecord(st.layer_ev[k], s) != cudaSuccess) return mfail(ELB_GENERAL_ERROR, "event record failed");
    int rc = (k > 0 && st.layers[k - 1].fused)
                 ? elb_conv_enqueue_strided(l.plan, y, x, st.layers[k - 1].d.oh, st.layers[k - 1].d.ow, st.layers[k - 1].step, s)
                 : elb_conv_enqueue(l.plan, y, x, nullptr, nullptr, s);
    if (rc != ELB_OK) return rc;
    x = y;
    if (l.step > 1 && !l.fused) {
      void *z = last ? output : l.d_sub;
      rc = elb_subsample_nChw16c(z, y, l.d.n, l.d.oc, l.d.oh, l.d.ow, l.step, l.step, (int)elem_bytes(l.d.dt_output), s);
      if (rc != ELB_OK) return rc;
      ++st.extra_launches;
      x = z;
    }
  }
  if (!st.layer_ev.empty() && cudaEventRecord(st.layer_ev[L], s) != cudaSuccess) return mfail(ELB_GENERAL_ERROR, "event record failed");
  return ELB_OK;
}

int stack_status(elb_stack &st) {
  for (size_t k = 0; k < st.layers.size(); ++k) {
    const int v = elb_conv_device_status(st.layers[k].plan);
    if (v != 0) return mfail(ELB_GENERAL_ERROR, "layer %d: device kernel gave up waiting (status %d)", (int)k, v);
  }
  return ELB_OK;
}

}  // namespace

extern "C" {

int elb_stack_create(const elb_conv_desc_t *descs, const int32_t *subsample_after, int n_layers, elb_stack_t **stack) {
  if (!descs || !stack || n_layers < 1) return mfail(ELB_GENERAL_ERROR, "null argument");
  *stack = nullptr;
  int dev = descs[0].device;
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) return mfail(ELB_GENERAL_ERROR, "no CUDA device available");
  elb_stack *st = new elb_stack();
  st->device = dev;
  st->n = descs[0].n;
  DevGuard guard(dev);
  for (int k = 0; k < n_layers; ++k) {
    elb_stack::Layer l;
    l.d = descs[k];
    l.d.device = dev;
    l.step = subsample_after ? subsample_after[k] : 1;
    if (l.step < 1) { delete st; return mfail(ELB_GENERAL_ERROR, "layer %d: subsample step must be >= 1", k); }
    if (l.d.fmt_input == ELB_FMT_UNDEF) l.d.fmt_input = ELB_NCHW16C;
    if (l.d.fmt_output == ELB_FMT_UNDEF) l.d.fmt_output = ELB_NCHW16C;
    // (the first layer may take the caller's plain image, nchw or nhwc, as the reference's own
    // first-layer runs do; everything between the layers is blocked)
    const bool plain_image = k == 0 && (l.d.fmt_input == ELB_NCHW || l.d.fmt_input == ELB_NHWC);
    if ((l.d.fmt_input != ELB_NCHW16C && !plain_image) || l.d.fmt_output != ELB_NCHW16C) {
      delete st;
      return mfail(ELB_UNIMPLEMENTED, "layer %d: a stack runs on nChw16c activations", k);
    }
    if (k > 0) {
      const elb_stack::Layer &p = st->layers[k - 1];
      const int ph = (p.d.oh + p.step - 1) / p.step, pw = (p.d.ow + p.step - 1) / p.step;
      if (l.d.n != p.d.n || l.d.ic != p.d.oc || l.d.ih != ph || l.d.iw != pw || l.d.dt_input != p.d.dt_output) {
        delete st;
        return mfail(ELB_GENERAL_ERROR, "layer %d does not take layer %d's output (n %d/%d, channels %d/%d, %dx%d/%dx%d, type %d/%d)",
                     k, k - 1, l.d.n, p.d.n, l.d.ic, p.d.oc, l.d.ih, l.d.iw, ph, pw, l.d.dt_input, p.d.dt_output);
      }
      if (l.d.with_ip_sum) { delete st; return mfail(ELB_UNIMPLEMENTED, "layer %d: in-place sum inside a stack", k); }
    }
    int rc = elb_conv_create(&l.d, &l.plan);
    if (rc != ELB_OK) { delete st; return rc; }
    elb_conv_info(l.plan, &l.info);
    st->layers.push_back(l);
  }
  // activation buffers between the layers
  for (int k = 0; k < n_layers; ++k) {
    elb_stack::Layer &l = st->layers[k];
    const bool last = k + 1 == n_layers;
    const size_t eb = elem_bytes(l.d.dt_output), ocp = (size_t)(l.d.oc + 15) / 16 * 16;
    const size_t sh = (l.d.oh + l.step - 1) / l.step, sw = (l.d.ow + l.step - 1) / l.step;
    const size_t sub_bytes = (size_t)l.d.n * ocp * sh * sw * eb;
    cudaError_t e = cudaSuccess;
    // a subsample in front of a layer that can read its input with a step costs nothing
    l.fused = l.step > 1 && !last && elb_conv_input_step_supported(st->layers[k + 1].plan) != 0;
    if (!last || l.step > 1) e = cudaMalloc(&l.d_out, l.info.bytes_output);
    if (e == cudaSuccess && l.step > 1 && !last && !l.fused) e = cudaMalloc(&l.d_sub, sub_bytes);
    if (e != cudaSuccess) { delete st; return mfail(ELB_GENERAL_ERROR, "device allocation failed: %s", cudaGetErrorString(e)); }
    if (last) st->out_bytes = l.step > 1 ? sub_bytes : l.info.bytes_output;
  }
  st->in_bytes = st->layers[0].info.bytes_input;
  if (cudaStreamCreateWithFlags(&st->s_run, cudaStreamNonBlocking) != cudaSuccess) {
    delete st;
    return mfail(ELB_GENERAL_ERROR, "stream creation failed");
  }
  *stack = st;
  return ELB_OK;
}

int elb_stack_prepare(elb_stack_t *stack, int layer, const void *weights, const void *bias) {
  if (!stack || layer < 0 || layer >= (int)stack->layers.size()) return mfail(ELB_GENERAL_ERROR, "bad layer index");
  int rc = elb_conv_prepare(stack->layers[layer].plan, weights, bias);
  if (rc == ELB_OK) stack->layers[layer].prepared = true;
  return rc;
}

int elb_stack_layer(elb_stack_t *stack, int layer, elb_conv_t **plan) {
  if (!stack || !plan || layer < 0 || layer >= (int)stack->layers.size()) return mfail(ELB_GENERAL_ERROR, "bad layer index");
  *plan = stack->layers[layer].plan;
  return ELB_OK;
}

int elb_stack_layer_output(elb_stack_t *stack, int layer, void **device_ptr, uint64_t *bytes) {
  if (!stack || !device_ptr || layer < 0 || layer >= (int)stack->layers.size()) return mfail(ELB_GENERAL_ERROR, "bad layer index");
  const elb_stack::Layer &l = stack->layers[layer];
  *device_ptr = l.d_out;          // null for the last layer: that tensor is the caller's
  if (bytes) *bytes = l.info.bytes_output;
  return ELB_OK;
}

int elb_stack_set_layer_events(elb_stack_t *stack, void **cuda_events, int count) {
  if (!stack) return mfail(ELB_GENERAL_ERROR, "null stack");
  stack->layer_ev.clear();
  if (!cuda_events) return ELB_OK;
  if (count != (int)stack->layers.size() + 1) return mfail(ELB_GENERAL_ERROR, "need one event per layer plus one");
  for (int i = 0; i < count; ++i) stack->layer_ev.push_back(static_cast<cudaEvent_t>(cuda_events[i]));
  return ELB_OK;
}

int elb_stack_sizes(const elb_stack_t *stack, int32_t *n_layers, uint64_t *bytes_input, uint64_t *bytes_output) {
  if (!stack) return mfail(ELB_GENERAL_ERROR, "null stack");
  if (n_layers) *n_layers = (int32_t)stack->layers.size();
  if (bytes_input) *bytes_input = stack->in_bytes;
  if (bytes_output) *bytes_output = stack->out_bytes;
  return ELB_OK;
}

uint64_t elb_stack_launch_count(const elb_stack_t *stack) {
  if (!stack) return 0;
  uint64_t n = stack->extra_launches;
  for (const auto &l : stack->layers) n += elb_conv_launch_count(l.plan);
  return n - stack->capture_counted + stack->graph_replays * stack->launches_per_chain;
}

int elb_stack_enqueue(elb_stack_t *stack, void *output, const void *input, void *cuda_stream) {
  if (!stack || !output || !input) return mfail(ELB_GENERAL_ERROR, "null argument");
  for (size_t k = 0; k < stack->layers.size(); ++k)
    if (!stack->layers[k].prepared) return mfail(ELB_GENERAL_ERROR, "layer %d has no weights yet (elb_stack_prepare)", (int)k);
  DevGuard guard(stack->device);
  return stack_enqueue(*stack, output, input, static_cast<cudaStream_t>(cuda_stream));
}

int elb_stack_execute(elb_stack_t *stack, void *output, const void *input, int64_t images) {
  if (!stack || !output || !input) return mfail(ELB_GENERAL_ERROR, "null argument");
  elb_stack &st = *stack;
  if (images <= 0 || images % st.n) return mfail(ELB_GENERAL_ERROR, "images must be a positive multiple of the stack's batch (%d)", st.n);
  for (size_t k = 0; k < st.layers.size(); ++k)
    if (!st.layers[k].prepared) return mfail(ELB_GENERAL_ERROR, "layer %d has no weights yet (elb_stack_prepare)", (int)k);
  DevGuard guard(st.device);
  const int64_t batches = images / st.n;
  const bool in_dev = on_device(input), out_dev = on_device(output);
  if (in_dev && out_dev) {
    for (int64_t b = 0; b < batches; ++b) {
      int rc = stack_enqueue(st, (uint8_t *)output + b * st.out_bytes, (const uint8_t *)input + b * st.in_bytes, st.s_run);
      if (rc != ELB_OK) { cudaStreamSynchronize(st.s_run); return rc; }
    }
    M_TRY(cudaStreamSynchronize(st.s_run));
    return stack_status(st);
  }
  // Host tensors: two staging slots.  While the chain works on slot b, the next batch is copied
  // into slot b^1 and the previous result leaves slot b^1 (three streams, two copy engines).  The
  // chain of a slot is captured ONCE into a CUDA graph (its tensors never move), so a batch costs
  // the host one graph launch instead of one launch per kernel.
  if (!st.s_h2d) {
    M_TRY(cudaStreamCreateWithFlags(&st.s_h2d, cudaStreamNonBlocking));
    M_TRY(cudaStreamCreateWithFlags(&st.s_d2h, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      M_TRY(cudaMalloc(&st.stage_in[i], st.in_bytes));
      M_TRY(cudaMalloc(&st.stage_out[i], st.out_bytes));
      M_TRY(cudaEventCreateWithFlags(&st.ev_in[i], cudaEventDisableTiming));
      M_TRY(cudaEventCreateWithFlags(&st.ev_run[i], cudaEventDisableTiming));
      M_TRY(cudaEventCreateWithFlags(&st.ev_out[i], cudaEventDisableTiming));
    }
  }
  for (int i = 0; i < 2 && i < batches; ++i) {
    if (st.graph[i]) continue;
    const uint64_t l0 = elb_stack_launch_count(stack);
    cudaGraph_t g = nullptr;
    M_TRY(cudaStreamBeginCapture(st.s_run, cudaStreamCaptureModeThreadLocal));
    int rc = stack_enqueue(st, st.stage_out[i], st.stage_in[i], st.s_run);
    cudaError_t e = cudaStreamEndCapture(st.s_run, &g);
    if (rc != ELB_OK) { if (g) cudaGraphDestroy(g); return rc; }
    if (e != cudaSuccess) return mfail(ELB_GENERAL_ERROR, "stream capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&st.graph[i], g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return mfail(ELB_GENERAL_ERROR, "graph instantiation failed: %s", cudaGetErrorString(e));
    st.launches_per_chain = elb_stack_launch_count(stack) - l0;
    st.capture_counted += st.launches_per_chain;
  }
  bool used[2] = {false, false};
  for (int64_t b = 0; b < batches; ++b) {
    const int i = (int)(b & 1);
    if (used[i]) {
      // slot i is free again when its previous chain has run (input) and its result has left (output)
      M_TRY(cudaStreamWaitEvent(st.s_h2d, st.ev_run[i], 0));
      M_TRY(cudaStreamWaitEvent(st.s_run, st.ev_out[i], 0));
    }
    const void *x = in_dev ? (const void *)((const uint8_t *)input + b * st.in_bytes) : nullptr;
    if (in_dev) M_TRY(cudaMemcpyAsync(st.stage_in[i], x, st.in_bytes, cudaMemcpyDeviceToDevice, st.s_h2d));
    else M_TRY(cudaMemcpyAsync(st.stage_in[i], (const uint8_t *)input + b * st.in_bytes, st.in_bytes, cudaMemcpyHostToDevice, st.s_h2d));
    M_TRY(cudaEventRecord(st.ev_in[i], st.s_h2d));
    M_TRY(cudaStreamWaitEvent(st.s_run, st.ev_in[i], 0));
    M_TRY(cudaGraphLaunch(st.graph[i], st.s_run));
    ++st.graph_replays;
    M_TRY(cudaEventRecord(st.ev_run[i], st.s_run));
    M_TRY(cudaStreamWaitEvent(st.s_d2h, st.ev_run[i], 0));
    M_TRY(cudaMemcpyAsync((uint8_t *)output + b * st.out_bytes, st.stage_out[i], st.out_bytes,
                          out_dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, st.s_d2h));
    M_TRY(cudaEventRecord(st.ev_out[i], st.s_d2h));
    used[i] = true;
  }
  M_TRY(cudaStreamSynchronize(st.s_run));
  M_TRY(cudaStreamSynchronize(st.s_d2h));
  return stack_status(st);
}

void elb_stack_destroy(elb_stack_t *stack) { delete stack; }

}  // extern "C"

// ================================================================================== multi-GPU
struct elb_conv_multi {
  struct Part {
    int device = 0, n0 = 0, cnt = 0;
    elb_conv_t *plan = nullptr;
  };
  std::vector<Part> parts;
  elb_conv_desc_t d{};
  elb_conv_info_t info{};      // of the whole batch
  size_t in_img = 0, out_img = 0;
  ~elb_conv_multi() {
    for (Part &p : parts) if (p.plan) elb_conv_destroy(p.plan);
  }
};

extern "C" {

int elb_conv_multi_create(const elb_conv_desc_t *desc, const int32_t *devices, int n_devices, elb_conv_multi_t **multi) {
  if (!desc || !multi) return mfail(ELB_GENERAL_ERROR, "null argument");
  *multi = nullptr;
  std::vector<int> devs;
  if (devices && n_devices > 0) {
    devs.assign(devices, devices + n_devices);
  } else {
    // EULER_GPUS = how many GPUs of this box share a minibatch (devices 0 .. G-1); default: all visible
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) { cudaGetLastError(); return mfail(ELB_GENERAL_ERROR, "no CUDA device available"); }
    int g = n_devices > 0 ? n_devices : count;
    if (const char *e = getenv("EULER_GPUS")) { const int v = atoi(e); if (v >= 1) g = v; }
    if (g > count) return mfail(ELB_GENERAL_ERROR, "%d GPUs asked for, %d visible", g, count);
    for (int i = 0; i < g; ++i) devs.push_back(i);
  }
  int G = (int)devs.size();
  if (G > desc->n) G = desc->n;           // fewer images than GPUs: the spare GPUs stay idle
  elb_conv_multi *m = new elb_conv_multi();
  m->d = *desc;
  int rc = elb_conv_sizes(desc, &m->info);
  if (rc != ELB_OK) { delete m; return rc; }
  m->in_img = m->info.bytes_input / desc->n;
  m->out_img = m->info.bytes_output / desc->n;
  for (int r = 0; r < G; ++r) {
    elb_conv_multi::Part p;
    p.device = devs[r];
    p.n0 = (int)((long long)desc->n * r / G);
    p.cnt = (int)((long long)desc->n * (r + 1) / G) - p.n0;
    elb_conv_desc_t d = *desc;
    d.n = p.cnt;
    d.device = p.device;
    rc = elb_conv_create(&d, &p.plan);
    if (rc != ELB_OK) { delete m; return rc; }
    m->parts.push_back(p);
  }
  *multi = m;
  return ELB_OK;
}

int elb_conv_multi_parts(const elb_conv_multi_t *multi, int32_t *n_parts, int32_t *devices, int32_t *first_image,
                         int32_t *image_count) {
  if (!multi || !n_parts) return mfail(ELB_GENERAL_ERROR, "null argument");
  const int cap = *n_parts;
  *n_parts = (int32_t)multi->parts.size();
  for (int r = 0; r < cap && r < (int)multi->parts.size(); ++r) {
    if (devices) devices[r] = multi->parts[r].device;
    if (first_image) first_image[r] = multi->parts[r].n0;
    if (image_count) image_count[r] = multi->parts[r].cnt;
  }
  return ELB_OK;
}

int elb_conv_multi_execute(elb_conv_multi_t *multi, void *output, const void *input, const void *weights, const void *bias) {
  if (!multi || !output || !input) return mfail(ELB_GENERAL_ERROR, "null argument");
  elb_conv_multi &m = *multi;
  if (on_device(input) || on_device(output))
    return mfail(ELB_GENERAL_ERROR, "elb_conv_multi_execute takes host tensors (one tensor of all N images)");
  // One host thread per GPU: each stages its slab of the host tensors through its own device
  // buffers (copy in, kernels and copy out overlapped per GPU as in elb_conv_execute) and the call
  // returns when every slab is back.  The slabs are disjoint, so nothing is exchanged.
  const size_t G = m.parts.size();
  std::vector<int> rcs(G, ELB_OK);
  std::vector<std::string> errs(G);
  auto work = [&](size_t r) {
    elb_conv_multi::Part &p = m.parts[r];
    cudaSetDevice(p.device);
    rcs[r] = elb_conv_execute(p.plan, (uint8_t *)output + (size_t)p.n0 * m.out_img,
                              (const uint8_t *)input + (size_t)p.n0 * m.in_img, weights, bias);
    if (rcs[r] != ELB_OK) errs[r] = elb_last_error();
  };
  std::vector<std::thread> th;
  for (size_t r = 1; r < G; ++r) th.emplace_back(work, r);
  {
    int prev = -1;
    cudaGetDevice(&prev);
    work(0);
    if (prev >= 0) cudaSetDevice(prev);
  }
  for (auto &t : th) t.join();
  for (size_t r = 0; r < G; ++r)
    if (rcs[r] != ELB_OK) return mfail(rcs[r], "GPU %d (images %d..%d): %s", m.parts[r].device, m.parts[r].n0,
                                       m.parts[r].n0 + m.parts[r].cnt - 1, errs[r].c_str());
  return ELB_OK;
}

void elb_conv_multi_destroy(elb_conv_multi_t *multi) { delete multi; }

}  // extern "C"
