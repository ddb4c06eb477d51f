#!/usr/bin/env python3
"""The reference arm of the benchmark: ling0322/libllm's own, unmodified code on the same GPU.

The reference is a C++/CUDA project without a Python package of its engine (``pip install`` of
its root finds no setup.py; its ``python/`` folder is a ctypes wrapper without the library), so
"installing" it means compiling it.  ``build()`` compiles, into ``baseline/_ref``:

* the reference's unmodified sources: ``src/lutil``, the CPU and CUDA parts of ``src/flint`` listed
  in ``src/flint/CMakeLists.txt:6-35`` and ``:55-83``, and the model files of ``src/libllm``, with the
  definitions its CMake gives for a CUDA build (``LIBLLM_CUDA_ENABLED``,
  ``LIBLLM_CUDA_MALLOC_ASYNC_ENABLED``; ``CMakeLists.txt:20-27``) for the architecture it lists for this
  GPU (``100-real``, ``CMakeLists.txt:42-45``).  FlashAttention is off (its sources are a download,
  ``third_party/install_flash_attn.sh``); attention then takes the reference's portable path
  (``src/flint/operators.cc:100-127``).  cuBLAS is opened by the reference itself with ``dlopen``
  (``src/flint/cuda/gemm_cublas.cc:123-130``);
* two files of our own: a stand-in for ``src/lutil/platform_linux.cc`` (which needs libunwind, a
  download) that defines the four functions of ``src/lutil/platform.h:29-32``, and a driver that
  builds ``LlamaModel`` from a tensor file on ``Device::getCuda()`` and times
  ``forward`` + ``forwardLmHead`` the way ``src/libllm/benchmark_main.cc:52-97`` and
  ``src/libllm/llama.cc:349-368`` call them, but with a device synchronisation on both sides of the
  timed region (the reference's own benchmark issues none).

``run()`` writes a tensor file of the benchmark's layer sizes with random float16 weights using the
reference's own writer (``tools/model_exporter.py``: ``TensorWriter``) under the reference's names
(``tools/llama_exporter.py:35-78``), runs the driver and returns its numbers.  None of this
repository's kernels, models or engine is on that path."""
from __future__ import annotations

import importlib.util
import json
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("LIBLLM_REFERENCE", "/root/reference")

PLATFORM_STANDIN = r"""
#include <stdint.h>
#include <stdlib.h>
#include "lutil/platform.h"
namespace lut {
void *alloc32ByteAlignedMem(int64_t nbytes) { void *p = nullptr; return posix_memalign(&p, 32, (nbytes + 31) / 32 * 32) ? nullptr : p; }
void free32ByteAlignedMem(void *p) { free(p); }
const char *getPathDelim() { return "/"; }
void printStackTrace() {}
}
"""

DRIVER = r"""
// usage: ref_bench model.bin hidden heads kv_heads intermediate eps layers vocab max_ctx prompt batch steps warmup
// prints one JSON object: prefill ms for `prompt` tokens, decode ms per step at `batch` (device-timed,
// token ids already on the device) and end to end (token ids from the host, sampled ids back to the host).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <chrono>
#include <memory>
#include <vector>
#include "flint/functional.h"
#include "flint/operators.h"
#include "libllm/kv_cache.h"
#include "libllm/llama.h"
#include "libllm/var_builder.h"
#include "lutil/reader.h"
using namespace libllm;
using namespace libllm::llama;
static double now() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
static void sync() {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { fprintf(stderr, "cuda: %s\n", cudaGetErrorString(e)); exit(3); }
}
static fl::Tensor ids(int batch, int len, int vocab, unsigned seed) {
  std::vector<fl::LongType> data((size_t)batch * len);
  for (auto &v : data) { seed = seed * 1664525u + 1013904223u; v = (fl::LongType)((seed >> 8) % (unsigned)vocab); }
  return fl::Tensor::create<fl::LongType>({batch, len}, data);
}
int main(int argc, char **argv) {
  if (argc != 14) return 2;
  fl::initOperators();
  const fl::Device dev = fl::Device::getCuda();
  auto reader = lut::ReadableFile::open(argv[1]);
  VarBuilder vb = VarBuilder::fromStream(reader.get(), dev, fl::DType::kFloat16);
  LlamaConfig cfg;
  cfg.hiddenSize = atoi(argv[2]);
  cfg.numHeads = atoi(argv[3]);
  cfg.numKeyValueHeads = atoi(argv[4]);
  cfg.intermediateSize = atoi(argv[5]);
  cfg.normEps = (float)atof(argv[6]);
  cfg.numLayers = atoi(argv[7]);
  cfg.vocabSize = atoi(argv[8]);
  cfg.maxContextLength = atoi(argv[9]);
  cfg.qkvProjBias = false;
  const int prompt = atoi(argv[10]), batch = atoi(argv[11]), steps = atoi(argv[12]), warmup = atoi(argv[13]);
  std::shared_ptr<LlamaModel> model = LlamaModel::build(cfg, vb.withName("llama"));
  sync();

  // prefill of one prompt: all positions through the layers, the last one through the output matrix
  // (src/libllm/llama.cc:349-357)
  double prefill_ms = 0;
  {
    fl::Tensor in = fl::F::to(dev, ids(1, prompt, cfg.vocabSize, 7));
    std::vector<double> times;
    for (int r = 0; r < 5; ++r) {
      KVCache past;
      sync();
      const double t0 = now();
      fl::Tensor x = model->forward(past, in);
      x = x.slice(1, {-1, fl::None});
      x = model->forwardLmHead(x);
      sync();
      if (r >= 2) times.push_back((now() - t0) * 1e3);
    }
    prefill_ms = times[times.size() / 2 > 0 ? 1 : 0];
    for (double t : times) if (t < prefill_ms) prefill_ms = t;       // best of three
  }

  // decode at `batch`: the prompts in one call, then one token each per step through the same KVCache
  // (src/libllm/llama.cc:359-368 for one sequence; the model's forward takes [N, T] ids)
  double step_ms = 0, e2e_ms = 0;
  {
    KVCache past;
    fl::Tensor x = model->forward(past, fl::F::to(dev, ids(batch, prompt, cfg.vocabSize, 11)));
    x = model->forwardLmHead(x.slice(1, {-1, fl::None}));
    sync();
    fl::Tensor one = fl::F::to(dev, ids(batch, 1, cfg.vocabSize, 13));
    for (int i = 0; i < warmup; ++i) model->forwardLmHead(model->forward(past, one));
    sync();
    double t0 = now();
    for (int i = 0; i < steps; ++i) model->forwardLmHead(model->forward(past, one));
    sync();
    step_ms = (now() - t0) * 1e3 / steps;
    // end to end: ids from host memory, the sampler's own path (src/libllm/generator.cc:197-214,
    // :113-121) with top_k 1, sampled ids back in host memory
    fl::Tensor host_ids = ids(batch, 1, cfg.vocabSize, 17);
    t0 = now();
    for (int i = 0; i < steps; ++i) {
      fl::Tensor in = fl::F::to(dev, host_ids);
      fl::Tensor logits = model->forwardLmHead(model->forward(past, in));
      fl::Tensor p = fl::F::softmax(logits.view({batch, cfg.vocabSize}));
      fl::Tensor sampled = fl::F::to(fl::Device::getCpu(), fl::F::sample(p, 1, 1.0f));
      const fl::LongType *s = sampled.getInternalData()->getData<fl::LongType>(sampled.getInternalOffset());
      fl::LongType *h = host_ids.getInternalData()->getData<fl::LongType>(host_ids.getInternalOffset());
      for (int b = 0; b < batch; ++b) h[b] = s[b];
    }
    sync();
    e2e_ms = (now() - t0) * 1e3 / steps;
  }
  printf("{\"prefill_ms\": %.4f, \"prefill_tokens\": %d, \"decode_ms_per_step\": %.4f, \"e2e_ms_per_step\": %.4f, "
         "\"batch\": %d, \"steps\": %d, \"warmup\": %d, \"context\": %d}\n",
         prefill_ms, prompt, step_ms, e2e_ms, batch, steps, warmup, prompt + warmup + 2 * steps);
  return 0;
}
"""

FLINT_CPU = """cpu/kernel/fallback.cc cpu/kernel/interface.cc cpu/kernel/util.cc cpu/all_close.cc cpu/binary_op.cc
cpu/cast.cc cpu/common.cc cpu/copy.cc cpu/cpu_operators.cc cpu/cpu_tensor_data.cc cpu/fill.cc cpu/lookup.cc
cpu/matmul.cc cpu/normalizations.cc cpu/print.cc cpu/rand.cc cpu/reduce.cc cpu/repetition_penalty.cc
cpu/softmax.cc cpu/swiglu.cc cpu/tensor.cc cpu/transform.cc cpu/view.cc device.cc dtype.cc functional.cc
operators.cc tensor.cc""".split()
FLINT_CUDA = """cuda/arange.cu cuda/binary.cu cuda/binary_scalar.cu cuda/cast.cu cuda/causal_mask.cu cuda/copy.cu
cuda/common.cc cuda/cuda_operators.cc cuda/cuda_tensor_data.cc cuda/dequant.cu cuda/fill.cu cuda/gemm_cublas.cc
cuda/lookup.cu cuda/matmul.cc cuda/matvec.cu cuda/print.cc cuda/rand.cc cuda/reduce.cu cuda/repetition_penalty.cu
cuda/rms_norm.cu cuda/sampling.cu cuda/softmax.cu cuda/swiglu.cu cuda/to_device.cc cuda/unary.cu""".split()
LIBLLM = "bpe generator kv_cache layers llama model_for_generation prompt tokenizer var_builder".split()
DEFINES = ["-DLIBLLM_CUDA_ENABLED", "-DLIBLLM_CUDA_MALLOC_ASYNC_ENABLED", "-D_FILE_OFFSET_BITS=64"]


def cuda_home() -> str:
    for base in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if base and os.path.isfile(os.path.join(base, "bin", "nvcc")):
            return base
    raise RuntimeError("nvcc not found")


def build(ref: str = REFERENCE, out: str = OUT) -> str:
    """Compiles the reference and the driver; returns the driver's path."""
    exe = os.path.join(out, "ref_bench")
    if os.path.isfile(exe):
        return exe
    if not os.path.isdir(os.path.join(ref, "src", "libllm")):
        raise RuntimeError(f"no checkout of ling0322/libllm at {ref}")
    objdir = os.path.join(out, "obj")
    os.makedirs(objdir, exist_ok=True)
    with open(os.path.join(out, "platform_standin.cc"), "w") as f:
        f.write(PLATFORM_STANDIN)
    with open(os.path.join(out, "driver.cc"), "w") as f:
        f.write(DRIVER)
    cuda = cuda_home()
    inc = ["-I", os.path.join(ref, "src"), "-I", os.path.join(ref, "third_party"), "-I", os.path.join(cuda, "include")]
    jobs = []   # (source, compiler argv)
    gxx = ["g++", "-std=c++17", "-O2", "-fopenmp"] + DEFINES + inc + ["-c"]
    nvcc = [os.path.join(cuda, "bin", "nvcc"), "-std=c++17", "-O3", "-gencode", "arch=compute_100,code=sm_100",
            "-DCUTE_ARCH_TCGEN05_TMEM_ENABLED", "--expt-relaxed-constexpr", "--use_fast_math",      # its own flags:
            "-Xcompiler", "-fopenmp"] + DEFINES + inc + ["-c"]                                   # src/flint/CMakeLists.txt:145
    for f in sorted(os.listdir(os.path.join(ref, "src/lutil"))):
        if f.endswith(".cc") and not f.endswith("_test.cc") and "windows" not in f and "darwin" not in f \
                and f != "platform_linux.cc":
            jobs.append((os.path.join(ref, "src/lutil", f), gxx))
    internal = os.path.join(ref, "src/lutil/internal")
    if os.path.isdir(internal):
        jobs += [(os.path.join(internal, f), gxx) for f in sorted(os.listdir(internal)) if f.endswith(".cc")]
    jobs += [(os.path.join(ref, "src/flint", f), gxx) for f in FLINT_CPU]
    jobs += [(os.path.join(ref, "src/flint", f), nvcc if f.endswith(".cu") else gxx) for f in FLINT_CUDA]
    jobs.append((os.path.join(ref, "src/flint/cpu/kernel/avx2.cc"), gxx[:-1] + ["-mavx2", "-mfma", "-mf16c", "-c"]))
    jobs.append((os.path.join(ref, "src/flint/cpu/kernel/avx512.cc"), gxx[:-1] + ["-mavx512f", "-c"]))
    jobs.append((os.path.join(ref, "third_party/ruapu/ruapu.cc"), gxx))
    jobs += [(os.path.join(ref, "src/libllm", f + ".cc"), gxx) for f in LIBLLM]
    jobs += [(os.path.join(out, "platform_standin.cc"), gxx), (os.path.join(out, "driver.cc"), gxx)]
    procs, objs = [], []
    limit = os.cpu_count() or 4

    def reap(src, p):
        err = p.communicate()[1]
        if p.returncode != 0:
            raise RuntimeError(f"compiling {src} failed:\n{err[-3000:]}")

    for i, (src, cmd) in enumerate(jobs):
        obj = os.path.join(objdir, f"o{i}.o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(cmd + [src, "-o", obj], stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True)))
        if len(procs) >= limit:
            reap(*procs.pop(0))
    for src, p in procs:
        reap(src, p)
    tmp = exe + ".tmp"
    subprocess.check_call(["g++", "-fopenmp", "-o", tmp] + objs + ["-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-lcurand",
                                                                     "-lpthread", "-ldl", "-lrt"])
    # the reference's own writer of its tensor file format travels with the install
    os.makedirs(os.path.join(out, "tools"), exist_ok=True)
    shutil.copy(os.path.join(ref, "tools", "model_exporter.py"), os.path.join(out, "tools", "model_exporter.py"))
    os.replace(tmp, exe)
    shutil.rmtree(objdir, ignore_errors=True)
    return exe


def reference_writer(out: str = OUT):
    spec = importlib.util.spec_from_file_location("ref_model_exporter", os.path.join(out, "tools", "model_exporter.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def rope_table(head_dim: int, theta: float, scaling, positions: int):
    """cos and sin [2, 1, positions, d] (the d/2 angles twice), the tensor the reference's exporter
    takes from the checkpoint's rotary module (tools/llama_exporter.py:54-62): for random weights any
    table times the same, so plain frequencies with the llama3 rule of the configuration."""
    import math
    import torch
    f = [theta ** (-2.0 * i / head_dim) for i in range(head_dim // 2)]
    if scaling:
        orig, lo, hi, fac = (float(scaling[k]) for k in ("original_max_position_embeddings", "low_freq_factor",
                                                          "high_freq_factor", "factor"))
        out = []
        for x in f:
            wl = 2 * math.pi / x
            if wl < orig / hi:
                out.append(x)
            elif wl > orig / lo:
                out.append(x / fac)
            else:
                s = (orig / wl - lo) / (hi - lo)
                out.append((1 - s) * x / fac + s * x)
        f = out
    angle = torch.arange(positions, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
    cos, sin = torch.cat([angle.cos(), angle.cos()], -1), torch.cat([angle.sin(), angle.sin()], -1)
    return torch.stack([cos, sin])[:, None, :, :].to(torch.float32)


def write_model(path: str, c: dict, max_ctx: int, seed: int = 0) -> None:
    """A tensor file of configuration ``c`` with random weights N(0, 0.02) and norm weights
    1 + U(-0.1, 0.1), float16, under the reference's names and fusions (tools/llama_exporter.py:35-78)."""
    import contextlib
    import io
    import torch
    mod = reference_writer()
    g = torch.Generator().manual_seed(seed)
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nH, nKV, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]

    def mat(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(torch.float16)

    def norm(n):
        return (1 + (torch.rand(n, generator=g) - 0.5) * 0.2).to(torch.float16)

    with contextlib.redirect_stdout(io.StringIO()):            # the writer prints a line per tensor
        with mod.TensorWriter(open(path, "wb")) as tw:
            emb = mat(V, H)
            tw.write_tensor(mod.Context("llama.embd.weight"), emb)
            tw.write_tensor(mod.Context("llama.norm.weight"), norm(H))
            tw.write_tensor(mod.Context("llama.rope"), rope_table(d, c["rope_theta"], c.get("rope_scaling"), max_ctx))
            tw.write_tensor(mod.Context("llama.out_proj.weight"), emb if c.get("tie_word_embeddings") else mat(V, H))
            for i in range(c["num_hidden_layers"]):
                q = f"llama.block{i}."
                tw.write_tensor(mod.Context(q + "input_norm.weight"), norm(H))
                tw.write_tensor(mod.Context(q + "post_attn_norm.weight"), norm(H))
                tw.write_tensor(mod.Context(q + "attn.qkv_proj.weight"), mat((nH + 2 * nKV) * d, H))
                tw.write_tensor(mod.Context(q + "attn.out_proj.weight"), mat(H, nH * d))
                tw.write_tensor(mod.Context(q + "mlp.gate_up_proj.weight"), mat(2 * I, H))
                tw.write_tensor(mod.Context(q + "mlp.down_proj.weight"), mat(H, I))


def run(c: dict, prompt: int, batch: int, steps: int, warmup: int, max_ctx: int, timeout: int = 1500) -> dict:
    """Builds (if need be), writes the model file to a temporary folder, runs the driver."""
    exe = build()
    with tempfile.TemporaryDirectory(prefix="libllm_ref_") as tmp:
        model = os.path.join(tmp, "model.bin")
        write_model(model, c, max_ctx)
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = os.path.join(cuda_home(), "lib64") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
        cmd = [exe, model, str(c["hidden_size"]), str(c["num_attention_heads"]), str(c["num_key_value_heads"]),
               str(c["intermediate_size"]), repr(c["rms_norm_eps"]), str(c["num_hidden_layers"]), str(c["vocab_size"]),
               str(max_ctx), str(prompt), str(batch), str(steps), str(warmup)]
        p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout)
    if p.returncode != 0:
        raise RuntimeError(f"the reference's driver exited with {p.returncode}: {(p.stderr or p.stdout)[-800:]}")
    return json.loads(p.stdout.strip().splitlines()[-1])


if __name__ == "__main__":
    print(build())
