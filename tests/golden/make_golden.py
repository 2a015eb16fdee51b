#!/usr/bin/env python3
"""Regenerate the golden vectors under tests/golden/ from a checkout of the reference.

Run where the reference tree is available (it is not needed to run the tests):

    python tests/golden/make_golden.py /path/to/ferrotensor

What it does
  1. imports the reference's own CPU restatement of the LoRA step,
     `scripts/gen_gradient_fixtures.py`, and runs its four cases in memory
     (nothing is written into the reference tree);
  2. checks the regenerated base weights and adapters bit for bit, and the
     regenerated loss / logits / gradients within 1e-4 + 1e-3*|e|, against the files
     the reference commits under
     `ferrotensor-graph/tests/fixtures/gradient_parity/`;
  3. writes `gradient_parity.npz`: config, weights, adapters, the cases and the
     reference's COMMITTED expected tensors (the authoritative numbers).

If `transformers` is importable it also runs `scripts/gen_qwen2_fixture.py` into a
temporary directory and stores its model, inputs, loss, logits and base-weight
gradients as `qwen2_family.npz` (q/k/v bias, tied embeddings, theta 1e6).
"""

import importlib.util
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
from safetensors.numpy import load_file

HERE = Path(__file__).resolve().parent


def load_module(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def gradient_parity(ref: Path):
    gen = load_module(ref / "scripts/gen_gradient_fixtures.py", "gen_gradient_fixtures")
    fx = ref / "ferrotensor-graph/tests/fixtures/gradient_parity"
    committed_model = load_file(fx / "model.safetensors")
    committed_adapters = load_file(fx / "adapters.safetensors")
    committed_expected = load_file(fx / "expected.safetensors")
    cases = json.loads((fx / "cases.json").read_text())
    config = json.loads((fx / "config.json").read_text())

    weights = gen.tiny_llama_weights()
    adapters = gen.make_adapters(weights)
    for n, v in weights.items():
        assert np.array_equal(v, committed_model[n]), f"weight {n} differs from the committed file"
    for n, v in adapters.items():
        assert np.array_equal(v, committed_adapters[n]), f"adapter {n} differs"

    worst = 0.0
    for case, spec in gen.CASES.items():
        p = {n: torch.tensor(v) for n, v in {**weights, **adapters}.items()}
        trainable = [n for n in p if n.endswith(".lora_a") or n.endswith(".lora_b")]
        if spec["trainable_base"]:
            trainable += [n for n in weights if n != "model.embed_tokens.weight"]
        for n in trainable:
            p[n].requires_grad_(True)
        ids = torch.tensor(spec["rows"], dtype=torch.long)
        logits = gen.forward(p, ids)
        loss = gen.loss_fn(logits, torch.tensor(spec["targets"]), torch.tensor(spec["masks"]))
        loss.backward()

        def check(name, got, exp):
            nonlocal worst
            err = np.abs(got - exp)
            tol = 1e-4 + 1e-3 * np.abs(exp)
            assert (err <= tol).all(), f"{case}/{name}: regenerated value off by {err.max()}"
            worst = max(worst, float(err.max()))

        check("loss", np.float32(loss.item()), np.float32(cases["cases"][case]["loss"]))
        check("logits", logits.detach().numpy(), committed_expected[f"logits.{case}"])
        for n in trainable:
            check(n, gen.ferrotensor_layout(n, p[n].grad).numpy(),
                  committed_expected[f"grad.{case}.{n}"])
    print(f"gradient_parity: regenerated == committed (worst abs diff {worst:.2e})")

    out = {"config_json": np.frombuffer(json.dumps(config).encode(), dtype=np.uint8),
           "cases_json": np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)}
    for n, v in committed_model.items():
        out[f"model/{n}"] = v
    for n, v in committed_adapters.items():
        out[f"adapter/{n}"] = v
    for n, v in committed_expected.items():
        out[f"expected/{n}"] = v
    np.savez_compressed(HERE / "gradient_parity.npz", **out)
    print(f"wrote {HERE / 'gradient_parity.npz'}")


def qwen2_family(ref: Path):
    try:
        import transformers  # noqa: F401
    except Exception as e:  # pragma: no cover
        print(f"qwen2_family skipped: transformers not importable ({e})")
        return
    import runpy
    with tempfile.TemporaryDirectory() as tmp:
        argv = sys.argv
        sys.argv = [str(ref / "scripts/gen_qwen2_fixture.py"), tmp]
        try:
            runpy.run_path(str(ref / "scripts/gen_qwen2_fixture.py"), run_name="__main__")
        finally:
            sys.argv = argv
        tmp = Path(tmp)
        out = {}
        model_dir = tmp / "model"
        out["config_json"] = np.frombuffer((model_dir / "config.json").read_bytes(), dtype=np.uint8)
        for n, v in load_file(model_dir / "model.safetensors").items():
            out[f"model/{n}"] = v
        for n, v in load_file(tmp / "expected.safetensors").items():
            out[f"expected/{n}"] = v
        out["cases_json"] = np.frombuffer((tmp / "cases.json").read_bytes(), dtype=np.uint8)
        np.savez_compressed(HERE / "qwen2_family.npz", **out)
        print(f"wrote {HERE / 'qwen2_family.npz'}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference repository>")
    ref = Path(sys.argv[1])
    gradient_parity(ref)
    qwen2_family(ref)
