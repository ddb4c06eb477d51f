#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ with ling0322/libllm's own CPU code.

    python tests/golden/make_golden.py --reference /path/to/libllm [--build DIR]

What it does, for the two tiny configurations of tests/golden/cases.py:
1. draws the weights (cases.py; rounded to float16, since the reference's tensor file
   stores 32-bit tensors as float16: tools/model_exporter.py:168-171),
2. writes them in the reference's tensor file format with the reference's own writer
   (tools/model_exporter.py, class TensorWriter) under the reference's names
   (tools/llama_exporter.py:35-78: stacked qkv_proj and gate_up_proj, out_proj, and the
   cos/sin table ``rope`` [2, 1, positions, d], which the reference does not compute:
   it is given OUR table, so the golden files anchor everything but the frequencies),
3. compiles the reference's CPU sources (src/lutil, the CPU part of src/flint listed in
   src/flint/CMakeLists.txt:6-35 and 103-122, and the model files of src/libllm) with g++,
   unmodified, plus two files of our own: a stand-in for src/lutil/platform_linux.cc
   (which needs libunwind, a download) that defines the four functions of
   src/lutil/platform.h:29-32, and a driver that builds LlamaModel from the file and runs
   forward + forwardLmHead as src/libllm/llama_test.cc:92-97 and :211-216 do,
4. runs the driver: logits of all positions for the whole prompt, and the logits of the
   last position after feeding the tokens one by one through one KVCache,
5. stores chosen rows of the logits as float32 in tests/golden/<case>.npz.

tests/test_golden.py compares tests/plain_llama.py with these files."""
import argparse
import importlib.util
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402

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
// usage: driver model.bin out.bin hidden heads kv_heads intermediate eps layers vocab max_ctx
#include <stdio.h>
#include <stdlib.h>
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
static fl::Tensor cpuFloat(fl::Tensor t) {
  return fl::F::contiguous(fl::F::cast(t, fl::DType::kFloat));
}
static void dump(FILE *fp, const fl::Tensor &t) {
  const float *p = t.getInternalData()->getData<float>(t.getInternalOffset());
  fwrite(p, sizeof(float), t.getNumEl(), fp);
}
int main(int argc, char **argv) {
  if (argc != 11) return 2;
  fl::initOperators();
  auto reader = lut::ReadableFile::open(argv[1]);
  VarBuilder vb = VarBuilder::fromStream(reader.get(), fl::Device::getCpu(), fl::DType::kFloat);
  LlamaConfig cfg;
  cfg.hiddenSize = atoi(argv[3]);
  cfg.numHeads = atoi(argv[4]);
  cfg.numKeyValueHeads = atoi(argv[5]);
  cfg.intermediateSize = atoi(argv[6]);
  cfg.normEps = (float)atof(argv[7]);
  cfg.numLayers = atoi(argv[8]);
  cfg.vocabSize = atoi(argv[9]);
  cfg.maxContextLength = atoi(argv[10]);
  cfg.qkvProjBias = false;
  std::shared_ptr<LlamaModel> model = LlamaModel::build(cfg, vb.withName("llama"));
  fl::Tensor ids = vb.getUnchecked("test_case.0.input_ids");
  int T = ids.getShape(0);
  FILE *fp = fopen(argv[2], "wb");
  {
    KVCache past;
    dump(fp, cpuFloat(model->forwardLmHead(model->forward(past, ids.view({1, T})))));
  }
  {
    KVCache past;
    fl::Tensor hidden;
    for (int i = 0; i < T; ++i) hidden = model->forward(past, ids.slice({i, i + 1}).view({1, 1}));
    dump(fp, cpuFloat(model->forwardLmHead(hidden)));
  }
  fclose(fp);
  return 0;
}
"""

FLINT = """cpu/kernel/fallback.cc cpu/kernel/interface.cc cpu/kernel/util.cc cpu/all_close.cc cpu/binary_op.cc
cpu/cast.cc cpu/common.cc cpu/copy.cc cpu/cpu_operators.cc cpu/cpu_tensor_data.cc cpu/fill.cc cpu/lookup.cc
cpu/matmul.cc cpu/normalizations.cc cpu/print.cc cpu/rand.cc cpu/reduce.cc cpu/repetition_penalty.cc
cpu/softmax.cc cpu/swiglu.cc cpu/tensor.cc cpu/transform.cc cpu/view.cc device.cc dtype.cc functional.cc
operators.cc tensor.cc""".split()
LIBLLM = "bpe generator kv_cache layers llama model_for_generation prompt tokenizer var_builder".split()


def build_driver(ref: str, build: str) -> str:
    os.makedirs(build, exist_ok=True)
    exe = os.path.join(build, "driver")
    if os.path.isfile(exe):
        return exe
    with open(os.path.join(build, "platform_standin.cc"), "w") as f:
        f.write(PLATFORM_STANDIN)
    with open(os.path.join(build, "driver.cc"), "w") as f:
        f.write(DRIVER)
    jobs = []   # (source, extra flags)
    for f in sorted(os.listdir(os.path.join(ref, "src/lutil"))):
        if f.endswith(".cc") and not f.endswith("_test.cc") and "windows" not in f and "darwin" not in f \
                and f != "platform_linux.cc":
            jobs.append((os.path.join(ref, "src/lutil", f), []))
    internal = os.path.join(ref, "src/lutil/internal")
    if os.path.isdir(internal):
        jobs += [(os.path.join(internal, f), []) for f in sorted(os.listdir(internal)) if f.endswith(".cc")]
    jobs += [(os.path.join(ref, "src/flint", f), []) for f in FLINT]
    jobs.append((os.path.join(ref, "src/flint/cpu/kernel/avx2.cc"), ["-mavx2", "-mfma", "-mf16c"]))
    jobs.append((os.path.join(ref, "src/flint/cpu/kernel/avx512.cc"), ["-mavx512f"]))
    jobs.append((os.path.join(ref, "third_party/ruapu/ruapu.cc"), []))
    jobs += [(os.path.join(ref, "src/libllm", f + ".cc"), []) for f in LIBLLM]
    jobs += [(os.path.join(build, "platform_standin.cc"), []), (os.path.join(build, "driver.cc"), [])]
    base = ["g++", "-std=c++17", "-O2", "-fopenmp", "-D_FILE_OFFSET_BITS=64", "-I", os.path.join(ref, "src"), "-I",
            os.path.join(ref, "third_party"), "-c"]
    procs, objs = [], []
    for i, (src, extra) in enumerate(jobs):
        obj = os.path.join(build, f"o{i}.o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(base + extra + [src, "-o", obj], stderr=subprocess.PIPE, text=True)))
        if len(procs) >= (os.cpu_count() or 4):
            src0, p = procs.pop(0)
            if p.wait() != 0:
                raise SystemExit(f"compiling {src0} failed:\n{p.stderr.read()}")
    for src0, p in procs:
        if p.wait() != 0:
            raise SystemExit(f"compiling {src0} failed:\n{p.stderr.read()}")
    subprocess.check_call(["g++", "-fopenmp", "-o", exe] + objs + ["-lpthread", "-ldl"])
    return exe


def reference_writer(ref: str):
    spec = importlib.util.spec_from_file_location("ref_model_exporter", os.path.join(ref, "tools/model_exporter.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def write_model_bin(mod, path: str, c: dict, w: dict, ids) -> None:
    """The reference's names and fusions (tools/llama_exporter.py:35-78)."""
    cos, sin = cases.rope_table(c)                                       # [positions, d] each
    rope = torch.stack([cos, sin])[:, None, :, :].to(torch.float32)      # [2, 1, positions, d]
    out = [("llama.embd.weight", w["model.embed_tokens.weight"]), ("llama.norm.weight", w["model.norm.weight"]),
           ("llama.rope", rope)]
    head = w["model.embed_tokens.weight"] if c["tie_word_embeddings"] else w["lm_head.weight"]
    out.append(("llama.out_proj.weight", head))
    for i in range(c["num_hidden_layers"]):
        p, q = f"model.layers.{i}.", f"llama.block{i}."
        out += [(q + "input_norm.weight", w[p + "input_layernorm.weight"]),
                (q + "post_attn_norm.weight", w[p + "post_attention_layernorm.weight"]),
                (q + "attn.qkv_proj.weight", torch.cat([w[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)),
                (q + "attn.out_proj.weight", w[p + "self_attn.o_proj.weight"]),
                (q + "mlp.gate_up_proj.weight", torch.cat([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]], 0)),
                (q + "mlp.down_proj.weight", w[p + "mlp.down_proj.weight"])]
    out.append(("test_case.0.input_ids", torch.tensor(ids, dtype=torch.int64)))
    with mod.TensorWriter(open(path, "wb")) as tw:
        for name, t in out:
            tw.write_tensor(mod.Context(name), t)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of ling0322/libllm")
    ap.add_argument("--build", default=os.path.join(tempfile.gettempdir(), "libllm_golden_build"))
    args = ap.parse_args()
    exe = build_driver(args.reference, args.build)
    mod = reference_writer(args.reference)
    for name, case in cases.CASES.items():
        c, ids = case["config"], case["ids"]
        w = cases.weights(c, case["seed"])
        model_bin = os.path.join(args.build, f"{name}.bin")
        out_bin = os.path.join(args.build, f"{name}.out")
        write_model_bin(mod, model_bin, c, w, ids)
        subprocess.check_call([exe, model_bin, out_bin, str(c["hidden_size"]), str(c["num_attention_heads"]),
                               str(c["num_key_value_heads"]), str(c["intermediate_size"]), repr(c["rms_norm_eps"]),
                               str(c["num_hidden_layers"]), str(c["vocab_size"]), str(c["max_position_embeddings"])])
        data = np.fromfile(out_bin, dtype="<f4")
        T, V = len(ids), c["vocab_size"]
        assert data.size == (T + 1) * V, (data.size, T, V)
        whole, last_by_token = data[:T * V].reshape(T, V), data[T * V:]
        rows = case["rows"]
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), rows=np.array(rows), logits=whole[rows].astype(np.float32),
                            last_token_by_token=last_by_token.astype(np.float32), checksum=np.array(cases.checksum(w)),
                            **{"w/" + k: t.numpy().astype(np.float16) for k, t in w.items()})
        print(f"{name}: {T} tokens, rows {rows}, max |whole[-1] - token by token| = "
              f"{np.abs(whole[-1] - last_by_token).max():.3e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
