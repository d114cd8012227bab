"""Model-level drop-in check: tiny random Hugging Face Llama (GQA) and OPT models with their linears
replaced by packed ones through `install_bitmap`, against the same model carrying the dequantised
weights.  Mirrors the reference's Crispybits/Kernel/tests/test_integration.py (prefill + four greedy
decode steps, fused QKV / gate-up, fused RoPE path, proxy misuse).  The CPU variants drive the package's
host logic with the oracle-backed stand-in; the GPU variants run the CUDA kernels.
"""
import copy

import pytest
import torch

transformers = pytest.importorskip("transformers")

import oracle_backend  # noqa: E402
from oracle import cb_oracle as O  # noqa: E402

from crispybits_kernels import FusedLlamaMLP, FusedQKV, install_bitmap, ops, tune_model  # noqa: E402
from crispybits_kernels.integration import _blocks  # noqa: E402


def _pack(m: torch.nn.Linear, bits, dtype):
    name = {torch.float16: "float16", torch.float32: "float32"}[dtype]
    d = O.pack_linear_dict(m.weight.detach().float().cpu().numpy(), bits, 128,
                           None if m.bias is None else m.bias.detach().float().cpu().numpy(), name)
    out = {k: (torch.from_numpy(v) if hasattr(v, "dtype") and not isinstance(v, (int, str)) else v) for k, v in d.items() if k != "dtype"}
    return d, out


def write_packed_dir(model, out_dir, bits_options, dtype):
    """The on-disk layout of Crispybits/Kernel/crispybits_kernels/reference.py:85-94."""
    for i, block in enumerate(_blocks(model)):
        linears = {n: m for n, m in block.named_modules() if isinstance(m, torch.nn.Linear)}
        for b in bits_options:
            torch.save({n: _pack(m, b, dtype)[1] for n, m in linears.items()}, out_dir / f"block_{i:03d}_w{b}.pt")


def dequantize_model_(model, bitmap, dtype):
    for block, bits in zip(_blocks(model), bitmap):
        for _, m in block.named_modules():
            if isinstance(m, torch.nn.Linear):
                d, _ = _pack(m, bits, dtype)
                m.weight.data.copy_(torch.from_numpy(O.dequantized_weight(d)).to(m.weight))


def tiny(kind):
    torch.manual_seed(0)
    if kind == "llama":
        cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=3,
                                       num_attention_heads=4, num_key_value_heads=2, vocab_size=512)
        model = transformers.LlamaForCausalLM(cfg)
        with torch.no_grad():      # sharper attention, so that a wrong rotation shows up in the logits
            for blk in _blocks(model):
                blk.self_attn.q_proj.weight.mul_(8.0)
                blk.self_attn.k_proj.weight.mul_(8.0)
        return model
    cfg = transformers.OPTConfig(hidden_size=256, ffn_dim=512, num_hidden_layers=3, num_attention_heads=4,
                                 vocab_size=512, word_embed_proj_dim=256)
    return transformers.OPTForCausalLM(cfg)


def run_model_check(env, tmp_path, kind, fuse, fuse_rope):
    dtype = torch.float16 if env == "cuda" else torch.float32
    base = tiny(kind).to(dtype).to(env).eval()
    bitmap = [4, 2, 3]
    write_packed_dir(base, tmp_path, (2, 3, 4), dtype)
    ref = copy.deepcopy(base)
    dequantize_model_(ref, bitmap, dtype)
    model = install_bitmap(copy.deepcopy(base), tmp_path, bitmap, device=env, dtype=dtype, fuse=fuse, fuse_rope=fuse_rope)
    if fuse and kind == "llama":
        owners = [m for m in model.modules() if isinstance(m, FusedQKV)]
        assert owners and any(isinstance(m, FusedLlamaMLP) for m in model.modules())
        assert all(bool(o.rope_head_dim) == fuse_rope for o in owners)
    if fuse:
        tuning = tune_model(model, iters=2, warmup=1, dtype=dtype)
        assert tuning and all({"split_k", "rho"} <= set(v) for v in tuning.values())
    ids = torch.randint(0, 512, (1, 12), device=env)
    with torch.no_grad():
        a, b = ref(ids, use_cache=True), model(ids, use_cache=True)
        la, lb = a.logits[:, -1], b.logits[:, -1]
        rel = (la.float() - lb.float()).abs().max() / la.float().abs().max()
        assert rel < 2e-2, f"prefill logits diverge: {rel:.3e}"
        pa, pb = a.past_key_values, b.past_key_values
        for _ in range(4):
            nxt = la.argmax(-1, keepdim=True)
            a, b = ref(nxt, past_key_values=pa, use_cache=True), model(nxt, past_key_values=pb, use_cache=True)
            la, lb, pa, pb = a.logits[:, -1], b.logits[:, -1], a.past_key_values, b.past_key_values
            rel = (la.float() - lb.float()).abs().max() / la.float().abs().max()
            assert rel < 2e-2, f"decode logits diverge: {rel:.3e}"


CASES = [("llama", False, False), ("llama", True, False), ("llama", True, True), ("opt", False, False), ("opt", True, True)]


@pytest.fixture
def oracle_env():
    prev = ops._C
    ops.set_backend(oracle_backend)
    ops._sm_count_for.cache_clear()
    yield "cpu"
    ops.set_backend(prev if prev is not None else "cuda")
    ops._sm_count_for.cache_clear()


@pytest.mark.parametrize("kind,fuse,fuse_rope", CASES)
def test_model_matches_dequantized_cpu(oracle_env, tmp_path, kind, fuse, fuse_rope):
    run_model_check("cpu", tmp_path, kind, fuse, fuse_rope)


@pytest.mark.gpu
@pytest.mark.parametrize("kind,fuse,fuse_rope", CASES)
def test_model_matches_dequantized_gpu(tmp_path, kind, fuse, fuse_rope):
    ops.set_backend("cuda")
    run_model_check("cuda", tmp_path, kind, fuse, fuse_rope)


def test_fused_rope_path_is_used_and_checked(oracle_env, tmp_path, monkeypatch):
    import sys
    from crispybits_kernels import integration
    dtype = torch.float32
    base = tiny("llama").to(dtype).eval()
    write_packed_dir(base, tmp_path, (3,), dtype)
    ref = copy.deepcopy(base)
    dequantize_model_(ref, [3, 3, 3], dtype)
    model = install_bitmap(copy.deepcopy(base), tmp_path, [3, 3, 3], device="cpu", dtype=dtype, fuse_rope=True)
    mod = sys.modules[type(_blocks(model)[0].self_attn).__module__]
    assert getattr(mod.apply_rotary_pos_emb, "_crispybits_patched", False)
    primes = []
    orig_prime = FusedQKV.prime
    monkeypatch.setattr(FusedQKV, "prime", lambda self, *a: (primes.append(1), orig_prime(self, *a))[1])
    ids = torch.randint(0, 512, (1, 16))

    def block0_update(m):
        h = m(ids, output_hidden_states=True).hidden_states
        return (h[1] - h[0]).float()

    with torch.no_grad():
        la, lb = block0_update(ref), block0_update(model)
    assert len(primes) == 3                       # one fused launch per block
    assert (la - lb).abs().max() / la.abs().max() < 2e-2
    for blk in _blocks(model):
        assert blk.self_attn.crispybits_qkv._cache is None
    monkeypatch.setattr(integration, "_mark", lambda t: t)     # without the mark the model rotates a second time
    with torch.no_grad():
        lb2 = block0_update(model)
    assert (la - lb2).abs().max() / la.abs().max() > 0.2


def test_proxy_mismatch_raises(oracle_env):
    from crispybits_kernels.integration import _QKVProxy
    from crispybits_kernels.ops import PackedLinear
    from helpers import make
    ws = [PackedLinear(make(128, 128, 3, torch.float32, "cpu", seed=s)[0]) for s in range(3)]
    ws[0].permute_for_rope_(64); ws[1].permute_for_rope_(64)
    owner = FusedQKV(*ws, rope_head_dim=64)
    x = torch.randn(1, 128)
    owner.prime(x, torch.ones(1, 64), torch.zeros(1, 64))
    with pytest.raises(RuntimeError):
        _QKVProxy(owner, 0)(x.clone())


def test_tuning_file_roundtrip(tmp_path):
    from crispybits_kernels import load_tuning, save_tuning
    t = {"block.0.self_attn.qkv": {"split_k": 2, "rho": 1}}
    save_tuning(t, str(tmp_path / "t.json"))
    assert load_tuning(str(tmp_path / "t.json")) == t and load_tuning(None) == {}
