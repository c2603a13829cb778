"""
Writes the golden files of this folder from tejkas/tinyserve-llm's own model code, on the CPU.

    python tests/golden/make_golden.py /path/to/tinyserve-llm

For tiny configurations A and B (tests/tiny_configs.py) it writes a model folder with this
repository's random-weights mode (seeded, so the tests regenerate the identical folder), loads it
with tinyserve-llm's loader into its LlamaForCausalLM (float32, CPU), and stores

  golden_<name>.json          token ids of the probe sequence, the rows kept, greedy continuations
                              that tinyserve-llm's LLM.generate produced, and inv_freq as hex floats
  golden_<name>_logits.npy    float32 logits [rows kept, vocab] of the probe sequence, computed with
                              tinyserve-llm's DenseCausalAttention oracle (whole sequence, no cache)

and, once,

  golden_parts_bf16.npz       what tinyserve-llm's own modules (RMSNorm with and without residual,
                              SiluAndMul, apply_rotary_emb) give in bfloat16 on the CPU for seeded
                              bfloat16 inputs: the places where its bfloat16 model rounds.  Logits of
                              a whole bfloat16 model cannot pin those places (one-ulp flips spread
                              chaotically through the layers: the plain float32 logits are as close
                              to tinyserve-llm's bfloat16 logits as the plain bfloat16 ones are), so
                              the parts are held to them one by one, bit for bit.

Nothing of tinyserve-llm is copied: it is imported, run once, and its small outputs are kept.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from tiny_configs import PAGE_A, PAGE_B, SEED_A, SEED_B, TINY_A, TINY_B, WEIGHTS  # noqa: E402

from tinyserve_llm_b200.weights import write_random_model  # noqa: E402


def probe_ids(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def main(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    os.environ["TINYSERVE_COMPILE"] = "0"
    from tinyserve_llm.engine.interface import CacheConfig
    from tinyserve_llm.engine.llm_engine import LLM
    from tinyserve_llm.model.attention import DenseCausalAttention
    from tinyserve_llm.model.loader import load_model
    from tinyserve_llm.scheduler.scheduler import SchedulerConfig
    from tinyserve_llm.scheduler.sequence import SamplingParams

    for name, raw, seed, page, length in (("a", TINY_A, SEED_A, PAGE_A, 60), ("b", TINY_B, SEED_B, PAGE_B, 200)):
        with tempfile.TemporaryDirectory() as folder:
            # stored in float32 so that tinyserve-llm's float32 model holds exactly the stored values
            write_random_model(folder, raw, seed, store_dtype="float32", **WEIGHTS)
            model = load_model(folder, dtype=torch.float32, device="cpu")
            ids = probe_ids(raw["vocab_size"], length, seed)
            with torch.no_grad():
                hidden = model(torch.tensor(ids), torch.arange(length), DenseCausalAttention([0, length]))
                logits = model.compute_logits(hidden).float()
            rows = sorted(set(range(0, length, 7)) | {length - 1})
            np.save(os.path.join(HERE, f"golden_{name}_logits.npy"), logits[rows].numpy())
            inv_freq = model.model.layers[0].self_attn.rotary_emb.inv_freq
            prompts = [ids[:5], ids[3:20], ids[10:43], ids[:40]]
            llm = LLM(folder, SchedulerConfig(max_model_len=128, max_num_seqs=8, max_num_batched_tokens=256,
                                              eos_token_id=-2),
                      CacheConfig(block_size=page, device="cpu"), dtype=torch.float32, num_blocks=64,
                      load_tokenizer=False)
            done = llm.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
            record = {
                "made_by": "tests/golden/make_golden.py from tinyserve-llm's LlamaForCausalLM (float32, CPU)",
                "config": raw,
                "seed": seed,
                "weights": WEIGHTS,
                "store_dtype": "float32",
                "ids": ids,
                "rows": rows,
                "inv_freq_hex": [float(x).hex() for x in inv_freq.tolist()],
                "prompts": prompts,
                "greedy": [c.token_ids[0] for c in done],
            }
            with open(os.path.join(HERE, f"golden_{name}.json"), "w") as f:
                json.dump(record, f)
            print(name, "logits", tuple(logits[rows].shape), "greedy", record["greedy"])


def parts_bf16(reference_root: str) -> None:
    sys.path.insert(0, reference_root)
    os.environ["TINYSERVE_COMPILE"] = "0"
    from tinyserve_llm.model.llama import RMSNorm, SiluAndMul, apply_rotary_emb

    g = torch.Generator().manual_seed(2024)
    bf = torch.bfloat16
    rows, hidden, inter, heads, hd = 6, 80, 48, 3, 16
    x = (3.0 * torch.randn(rows, hidden, generator=g)).to(bf)
    residual = (3.0 * torch.randn(rows, hidden, generator=g)).to(bf)
    weight = (1.0 + 0.25 * torch.randn(hidden, generator=g)).to(bf)
    gate_up = (2.0 * torch.randn(rows, 2 * inter, generator=g)).to(bf)
    q = torch.randn(rows, heads, hd, generator=g).to(bf)
    angles = torch.rand(rows, 1, hd // 2, generator=g) * 50.0
    cos, sin = angles.cos(), angles.sin()
    eps = 1e-5
    norm = RMSNorm(hidden, eps).to(bf)
    with torch.no_grad():
        norm.weight.copy_(weight)
        plain_norm = norm(x)
        added, carried = norm(x, residual)
        act = SiluAndMul()(gate_up)
        rotated = apply_rotary_emb(q, cos, sin)
    as32 = lambda t: t.float().numpy()       # noqa: E731  (bfloat16 values are exact in float32)
    np.savez(os.path.join(HERE, "golden_parts_bf16.npz"), eps=np.float64(eps), x=as32(x), residual=as32(residual),
             weight=as32(weight), rms_norm=as32(plain_norm), add_rms_norm=as32(added), carried=as32(carried),
             gate_up=as32(gate_up), swiglu=as32(act), q=as32(q), cos=cos.numpy(), sin=sin.numpy(),
             rotated=as32(rotated))
    print("parts in bfloat16 written")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <folder of tinyserve-llm's source tree>")
    main(sys.argv[1])
    parts_bf16(sys.argv[1])
