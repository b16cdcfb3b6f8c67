"""Generates tests/golden/reference_vectors.pt by running the REFERENCE's own PyTorch path
(triton_kernels.flux.layers and triton_kernels.functional, imported from a checkout of
ai-compiler-study/triton-kernels) on the seeded inputs of cases.py.

Usage:  python tests/golden/make_golden.py /path/to/triton-kernels-checkout

The reference is needed only to (re)generate the file; the tests read the committed file.
Outputs are float32 on CPU.  Each case also stores a fingerprint of its inputs so a test can
tell an RNG mismatch from a numerical one.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases  # noqa: E402


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    import triton_kernels.flux.layers as ref
    from triton_kernels.functional import apply_rope_torch, layer_norm_modulation_torch, rms_norm_torch

    torch.manual_seed(0)
    out: dict = {}

    def fp(d):
        return {k: cases.fingerprint(v) for k, v in d.items() if isinstance(v, torch.Tensor)}

    c = cases.case_rms_norm()
    out["rms_norm"] = {"y": rms_norm_torch(c["x"], c["scale"]), "y_module": None, "fp": fp(c)}
    m = ref.RMSNorm(128)
    m.load_state_dict({"scale": c["scale"]})
    out["rms_norm"]["y_module"] = m(c["x"]).detach()

    c = cases.case_layer_norm_modulation()
    out["layer_norm_modulation"] = {"y": layer_norm_modulation_torch(c["x"], c["scale"], c["shift"]), "fp": fp(c)}

    c = cases.case_rope_random_table()
    q, k = apply_rope_torch(c["q"], c["k"], c["pe"])
    q2, k2 = ref.apply_rope(c["q"], c["k"], c["pe"])
    assert torch.equal(q, q2) and torch.equal(k, k2)
    out["rope_random_table"] = {"q": q, "k": k, "fp": fp(c)}

    c = cases.case_embed_nd()
    pe = ref.EmbedND(128, c["theta"], c["axes_dim"])(c["ids"])
    out["embed_nd"] = {"pe": pe}

    c = cases.case_timestep_embedding()
    out["timestep_embedding"] = {"emb": ref.timestep_embedding(c["t"], c["dim"])}

    c = cases.case_mlp_embedder()
    m = ref.MLPEmbedder(256, 256)
    m.load_state_dict(c["params"])
    out["mlp_embedder"] = {"y": m(c["x"]).detach(), "fp": fp(c)}

    def run_single(c):
        blk = ref.SingleStreamBlock(c["hidden"], c["heads"], 4.0)
        blk.load_state_dict(c["params"])
        pe = ref.EmbedND(128, 10000, [16, 56, 56])(c["ids"])
        with torch.no_grad():
            return blk(c["x"], c["vec"], pe)

    c = cases.case_single_block_small()
    out["single_block_small"] = {"y": run_single(c), "fp": fp({"x": c["x"], "w": c["params"]["linear1.weight"]})}

    c = cases.case_double_block_small()
    blk = ref.DoubleStreamBlock(c["hidden"], c["heads"], 4.0)
    blk.load_state_dict(c["params"])
    pe = ref.EmbedND(128, 10000, [16, 56, 56])(c["ids"])
    with torch.no_grad():
        img, txt = blk(c["img"], c["txt"], c["vec"], pe)
    out["double_block_small"] = {"img": img, "txt": txt, "fp": fp({"img": c["img"], "w": c["params"]["img_mlp.0.weight"]})}

    c = cases.case_last_layer()
    m = ref.LastLayer(c["hidden"], 1, c["out"])
    m.load_state_dict(c["params"])
    with torch.no_grad():
        out["last_layer"] = {"y": m(c["x"], c["vec"]), "fp": fp({"x": c["x"]})}

    # Benchmark config 1 at full size; only a strided sample and summary statistics are kept.
    c = cases.case_single_block_config1()
    y = run_single(c)
    out["single_block_config1"] = {
        "sample": y[0, ::16, ::48].contiguous(),
        "stats": torch.tensor([float(y.mean()), float(y.std()), float(y.abs().max())]),
        "fp": fp({"x": c["x"], "w": c["params"]["linear1.weight"]}),
    }

    torch.save(out, HERE / "reference_vectors.pt")
    total = sum(t.numel() for d in out.values() for t in d.values() if isinstance(t, torch.Tensor))
    print(f"wrote {HERE / 'reference_vectors.pt'}: {len(out)} cases, {total} floats")


if __name__ == "__main__":
    main(sys.argv[1])
