"""Makes tests/golden/tiny_r_reference.npz and tiny_r2_reference.npz: logits of kurulav1/cpi's own, unmodified
Llama4 CPU engine on the tiny configurations "R" and "R2" (tests/tiny.py), for comparison with
tests/plain_llama4.py.

    python tests/golden/make_golden.py REFERENCE_ROOT        (a checkout of kurulav1/cpi)

It compiles src/engine/llama4_cpu_engine.cpp, src/model/safetensors_loader.cpp and
src/platform/mmap_file.cpp of the reference with ref_harness.cpp (g++, CUDA headers only, no CUDA
library), writes the tiny model to a temporary folder, runs the harness token by token and stores the
tokens, the logits at every position and a digest of the weights.  The random weights come from the
library's counter-based generator (integer mixing and a table look-up), so they do not depend on torch's
own generators; should the digest differ all the same (the table's last bits, from another erfinv), the test
skips rather than fails: run this script again.
"""
import hashlib
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import tiny  # noqa: E402


def weights_digest(model_dir):
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py REFERENCE_ROOT")
    ref = sys.argv[1]
    work = tempfile.mkdtemp(prefix="cpi_golden_")
    exe = os.path.join(work, "ref_harness")
    srcs = [os.path.join(ref, p) for p in ("src/engine/llama4_cpu_engine.cpp", "src/model/safetensors_loader.cpp",
                                           "src/platform/mmap_file.cpp")]
    cmd = ["g++", "-std=c++20", "-O2", "-mavx2", "-mfma", "-fopenmp", f"-I{ref}/include",
           "-I/usr/local/cuda/include", os.path.join(HERE, "ref_harness.cpp"), *srcs, "-o", exe]
    subprocess.run(cmd, check=True)
    for name, n_tokens, file in (("R", 48, "tiny_r_reference.npz"), ("R2", 70, "tiny_r2_reference.npz")):
        d = tiny.make_model_dir(name)
        c = tiny.config(name)["text_config"]
        rs = c["rope_scaling"]
        tokens = tiny.random_tokens(n_tokens, c["vocab_size"], 77)
        out = os.path.join(work, f"logits_{name}.f32")
        args = [exe, d, out, c["vocab_size"], c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"],
                c["head_dim"], c["num_hidden_layers"], c["num_local_experts"], c["intermediate_size"],
                c["intermediate_size"], rs["original_max_position_embeddings"], c["rope_theta"], rs["factor"],
                rs["low_freq_factor"], rs["high_freq_factor"], *tokens]
        subprocess.run([str(a) for a in args], check=True)
        logits = np.fromfile(out, dtype="<f4").reshape(len(tokens), c["vocab_size"])
        np.savez_compressed(os.path.join(HERE, file), tokens=np.array(tokens, dtype=np.int32),
                            logits=logits.astype(np.float32), digest=np.array(weights_digest(d)))
        print("wrote", file, logits.shape, "max |logit|", float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
