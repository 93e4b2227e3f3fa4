"""Runs the reference's own language model (NickWilde18/oxr-inference, ``oxr_runtime/language.py``) on the CPU in
fp32 on a tiny random Qwen3 model and stores its logits next to the weights and token ids that produced them:
``reference_tiny.safetensors``. ``tests/test_plain.py`` checks the plain implementation against that file.

How the reference is driven: ``tests/test_language_fused.py`` of the reference installs a pure-PyTorch stand-in
for its attention module when imported (lines 17-65), after which ``LanguageModel`` runs on CPU tensors; its
Triton kernel has a PyTorch twin for CPU inputs (``oxr_runtime/kernels.py:110-113``). The page size, a module
constant of 256, is set to 8 in both modules that hold it. 23 tokens are prefilled in one batch, the other 9
are decoded one by one, so the stored logits exercise both of the reference's forward passes.

Usage (needs the reference checkout; nothing else in the test suite does):

    python tests/golden/make_reference_golden.py /path/to/oxr-inference
"""

import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 32, "intermediate_size": 48, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "vocab_size": 61, "tie_word_embeddings": False, "max_position_embeddings": 64,
}
PREFILL, TOTAL, PAGE = 23, 32, 8


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "tests"))
    sys.path.insert(0, reference_root)
    import test_language_fused  # noqa: F401  installs the attention stand-in before oxr_runtime.language is imported
    from oxr_runtime import kv_cache, language
    from oxr_runtime.config import LanguageConfig

    kv_cache.BLOCK_SIZE = language.BLOCK_SIZE = PAGE
    c = LanguageConfig(hidden_size=32, intermediate_size=48, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                       rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=61)
    torch.manual_seed(1234)
    model = language.LanguageModel(c, max_positions=64)
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(1 + 0.1 * torch.randn_like(p) if "norm" in name else 0.2 * torch.randn_like(p))
    model = model.float().eval().requires_grad_(False)
    # checkpoint names: the reference's module names are the checkpoint's with the sub-module level removed
    # (oxr_runtime/weight_names.py:25-32)
    weights = {}
    for name, p in model.named_parameters():
        parts = name.split(".")
        if parts[0] == "layers":
            leaf = ".".join(parts[2:])
            if leaf.split(".")[0] in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm"):
                leaf = "self_attn." + leaf
            elif leaf.split(".")[0] in ("gate_proj", "up_proj", "down_proj"):
                leaf = "mlp." + leaf
            weights[f"model.layers.{parts[1]}.{leaf}"] = p.detach().clone()
        elif parts[0] == "lm_head":
            weights["lm_head.weight"] = p.detach().clone()
        else:
            weights["model." + name] = p.detach().clone()
    model.cast_rope(torch.float32)
    model.fuse_projections()

    ids = torch.randint(0, c.vocab_size, (TOTAL,), generator=torch.Generator().manual_seed(99))
    cache = kv_cache.KVCache(c, num_blocks=TOTAL // PAGE + 1, dtype=torch.float32, device=torch.device("cpu"))
    blocks = cache.allocate(kv_cache.blocks_for(TOTAL))
    rows = []
    with torch.inference_mode():
        batch = language.PrefillBatch(
            model.embed_tokens(ids[:PREFILL]), torch.arange(PREFILL), torch.tensor([0, PREFILL], dtype=torch.int32), PREFILL,
            torch.tensor([language.slot_of(blocks, p) for p in range(PREFILL)]))
        rows.append(model.logits(model.prefill(batch, cache)))
        for p in range(PREFILL, TOTAL):
            step = language.DecodeBatch(
                model.embed_tokens(ids[p:p + 1]), torch.tensor([p]), torch.tensor([language.slot_of(blocks, p)]),
                torch.tensor([p + 1], dtype=torch.int32), torch.tensor([blocks], dtype=torch.int32))
            rows.append(model.logits(model.decode(step, cache)))
    out = {k: v.contiguous() for k, v in weights.items()}
    out["golden.token_ids"] = ids.to(torch.int32)
    out["golden.reference_logits"] = torch.cat(rows).float().contiguous()
    save_file(out, str(HERE / "reference_tiny.safetensors"))
    print(f"wrote {HERE / 'reference_tiny.safetensors'}: logits {tuple(out['golden.reference_logits'].shape)}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_reference_golden.py /path/to/oxr-inference")
    main(sys.argv[1])
