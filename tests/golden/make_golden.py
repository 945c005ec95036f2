"""Compare the plain implementation (tests/plain_qwen3.py) with the reference's own
model code once, on tiny random models, and store the small outputs.

Run from the repository root, on a machine that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's dense-cache model (model/qwen/qwen_kv_cont.py Qwen3, which
masks `k_pos <= position` and therefore also handles a prompt fed in portions), loads
the random weights of tiny models A and B0 into it (for the untied B0 the reference
has no lm_head: its final-norm output is hooked and multiplied with lm_head here),
feeds one sequence whole, and writes `golden_<name>.pt` with the configuration, the
token ids and the reference's float32 logits at a few positions, and
`golden_<name>.safetensors` with the very weights it ran (a few hundred KB), so that
the comparison does not depend on which random numbers this machine's torch draws.  The
test tests/test_plain.py::test_plain_matches_reference_golden recomputes those logits
with the plain implementation.  The reference's code is only imported and run, never copied.
"""

import hashlib
import os
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def weights_checksum(w):
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(k.encode())
        h.update(w[k].to(torch.float32).numpy().tobytes())
    return h.hexdigest()


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = sys.argv[1]
    os.environ["HF_HUB_OFFLINE"] = "1"
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref)
    from model.qwen.qwen_kv_cont import KVCache, Qwen3      # the reference's classes

    import plain_qwen3 as plain
    from tiny_configs import make_folder

    out_dir = Path(__file__).resolve().parent
    for name in ("A", "B0"):
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_folder(Path(tmp), name)
            cfg, w = plain.load_folder(folder)
        sd = {k.removeprefix("model."): v.float() for k, v in w.items() if k != "lm_head.weight"}
        model = Qwen3(cfg).float().eval()
        model.load_state_dict(sd)
        n = 45
        g = torch.Generator().manual_seed(1234)
        ids = torch.randint(0, cfg["vocab_size"], (1, n), generator=g)
        model.attach_cache(KVCache(1, cfg["num_hidden_layers"], cfg["num_key_value_heads"],
                                   cfg["head_dim"], max_len=64, dtype=torch.float32, device="cpu"))
        hidden = {}
        model.norm.register_forward_hook(lambda m, i, o: hidden.__setitem__("h", o))
        with torch.no_grad():
            logits = model(ids, slice(0, 1), torch.arange(n)[None], n)[0]
        if not cfg.get("tie_word_embeddings", False):
            logits = hidden["h"][0] @ w["lm_head.weight"].float().T
        keep = [0, 1, 15, 16, 17, 31, 44]
        mine = plain.logits(w, cfg, ids[0].tolist(), torch.float32)
        print(name, "max |plain - reference| =", (mine - logits).abs().max().item(),
              "max |reference| =", logits.abs().max().item())
        from safetensors.torch import save_file
        save_file({k: v.contiguous() for k, v in w.items()}, str(out_dir / f"golden_{name}.safetensors"))
        torch.save({"config": cfg, "ids": ids[0].tolist(), "positions": keep, "logits": logits[keep].clone(),
                    "weights_sha256": weights_checksum(w)}, out_dir / f"golden_{name}.pt")


if __name__ == "__main__":
    main()
