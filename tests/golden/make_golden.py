"""Makes tests/golden/reference_logits_tiny_a.json.

Builds the reference's CPU library out of tree (cmake, no CUDA), compiles
tests/golden/golden_driver.cpp against it, runs a tiny Llama (2 layers, hidden 64, 4 heads,
2 KV heads, head size 16, feed-forward 176, vocabulary 256: the sizes whose constants the
reference fixes in code, theta 10000 and eps 1e-5) through the reference's own classes for
three prompts, and stores the logits of every position.

    python tests/golden/make_golden.py PATH_OF_THE_REFERENCE_CHECKOUT
"""
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from golden_model import CONFIG, golden_weights  # noqa: E402

SEED = 20240611
PROMPT_LENGTHS = (5, 9, 13)


def main():
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    reference = Path(sys.argv[1])
    work = Path(tempfile.mkdtemp(prefix="stratakv_golden_"))
    build = work / "build"
    subprocess.run(["cmake", "-S", str(reference), "-B", str(build), "-DSTRATAKV_CUDA=OFF",
                    "-DCMAKE_BUILD_TYPE=Release"], check=True, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", str(build), "--target", "stratakv", "-j", "8"], check=True,
                   stdout=subprocess.DEVNULL)
    library = next(build.rglob("libstratakv.a"))
    driver = work / "golden_driver"
    subprocess.run(["g++", "-std=c++17", "-O2", "-mavx2", "-mfma", "-I", str(reference / "include"),
                    str(HERE / "golden_driver.cpp"), str(library), "-lpthread", "-o", str(driver)], check=True)
    weights = golden_weights(CONFIG, SEED)
    raw = work / "weights"
    raw.mkdir()
    for name, tensor in weights.items():
        (raw / f"{name}.f32").write_bytes(tensor.contiguous().numpy().astype("<f4").tobytes())
    generator = torch.Generator().manual_seed(SEED + 1)
    cases = []
    for length in PROMPT_LENGTHS:
        tokens = torch.randint(0, CONFIG["vocab_size"], (length,), generator=generator).tolist()
        c = CONFIG
        out = subprocess.run([str(driver), str(raw), str(c["num_hidden_layers"]), str(c["hidden_size"]),
                              str(c["intermediate_size"]), str(c["num_attention_heads"]),
                              str(c["num_key_value_heads"]), str(c["vocab_size"]), *map(str, tokens)],
                             check=True, capture_output=True, text=True).stdout
        logits = [float(line) for line in out.split()]
        assert len(logits) == length * c["vocab_size"]
        cases.append({"tokens": tokens, "logits": logits})
    golden = {"made_by": "tests/golden/make_golden.py", "reference": "Mourya05/StrataKV CPU classes "
              "(TransformerBlock, RMSNorm, Linear, BlockPool, PageTable), float32 weights",
              "config": CONFIG, "seed": SEED,
              "weights_abs_sum": float(sum(float(w.double().abs().sum()) for w in weights.values())),
              "cases": cases}
    (HERE / "reference_logits_tiny_a.json").write_text(json.dumps(golden))
    print(f"wrote {HERE / 'reference_logits_tiny_a.json'} ({sum(len(c['logits']) for c in cases)} logits)")


if __name__ == "__main__":
    main()
