"""Packaging (.aio), chat session, sampler and stream renderer on CPU."""
import io
import json
import os
import subprocess
import sys

import pytest
import torch

from loomformer_paraplex_b200.config import Config
from loomformer_paraplex_b200.data.tokenizers import BPETokenizer, train_tokenizer
from loomformer_paraplex_b200.models.loomformer import Model
from loomformer_paraplex_b200.serve import chat as ch
from loomformer_paraplex_b200.serve import package as pk
from loomformer_paraplex_b200.train import checkpoint as ckpt

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORDS = "alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu".split()


@pytest.fixture(scope="module")
def packed(tmp_path_factory):
    d = tmp_path_factory.mktemp("pack")
    tokp = str(d / "tok.json")
    train_tokenizer("", 320, tokp, texts=[" ".join(WORDS)] * 50)
    tok = BPETokenizer.load(tokp)
    cfg = Config(vocab=tok.vocab_size, tokenizer=tokp, seq_len=96, model_dim=64, n_q_heads=4, n_kv_heads=2, hidden=1024,
                 layers=2, activation="pvpowlu", tria_carry_enabled=True, tria_temporal_auto=False,
                 tria_temporal_window=16, tied_embeddings=True)
    torch.manual_seed(0)
    model = Model(cfg)
    ckpt.save_checkpoint(str(d / "m.pt"), cfg, model, None, "adamw", 3, 123)
    return d, tok, cfg, model


def test_pack_quantises_only_large_matrices_and_keeps_aliases(packed):
    d, tok, cfg, model = packed
    out = str(d / "m.aio")
    man = pk.build_package(str(d / "m.pt"), str(d / "tok.json"), os.path.join(ROOT, "chat_template.jinja"), out, "bf16",
                           min_quant_elements=4096)
    pkg = pk.load_aio(out)
    st = pkg["checkpoint"]["model"]
    assert pkg["format"] == "loom.aio" and pkg["version"] == 1 and "optimizer" not in pkg["checkpoint"]
    assert st["emb.weight"].dtype == torch.bfloat16
    assert st["emb.weight"].data_ptr() == st["head.weight"].data_ptr()          # tie survives packing
    for name, t in st.items():
        if t.is_floating_point() and (t.ndim < 2 or "norm" in name or "beta_anchor" in name or name.endswith(".bias")):
            assert t.dtype == torch.float32, name
    q = man["quantization"]
    assert q["changed_tensors"] > 0 and q["packed_tensor_bytes"] < q["source_bytes"] and q["decisions"]["alias"] == 1
    assert man["assets"]["tokenizer"]["bytes"] == os.path.getsize(d / "tok.json")
    with pytest.raises(ValueError):
        pk.parse_quant("int3")


def test_pack_cli_roundtrip_and_reference_reads_it(packed):
    d, *_ = packed
    env = dict(os.environ, PYTHONPATH=ROOT)
    tool = os.path.join(ROOT, "loompack.py")
    r = subprocess.run([sys.executable, tool, "pack", "m.pt", "--tokenizer", "tok.json", "--template",
                        os.path.join(ROOT, "chat_template.jinja"), "-o", "cli.aio", "--quant", "fp16"], cwd=d, env=env,
                       capture_output=True, text=True)
    assert r.returncode == 0 and "[loompack] cli.aio:" in r.stdout and "quant=fp16" in r.stdout, r.stderr
    r = subprocess.run([sys.executable, tool, "inspect", "cli.aio", "--keys"], cwd=d, env=env, capture_output=True, text=True)
    assert '"format": "loom.aio"' in r.stdout and "emb.weight" in r.stdout
    r = subprocess.run([sys.executable, tool, "extract", "cli.aio", "-d", "x"], cwd=d, env=env, capture_output=True, text=True)
    assert r.returncode == 0 and sorted(os.listdir(d / "x")) == ["chat_template.jinja", "manifest.json", "model.pt", "tokenizer.json"]
    r = subprocess.run([sys.executable, tool, "inspect", "m.pt"], cwd=d, env=env, capture_output=True, text=True)
    assert r.returncode == 1 and "loompack:" in r.stderr
    # the reference's own loader accepts the archive
    ref = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(ref):
        code = ("import sys; sys.path.insert(0, %r); import loompack; p = loompack.load_aio('cli.aio'); "
                "print(p['manifest']['model']['state_keys'])" % ref)
        r = subprocess.run([sys.executable, "-c", code], cwd=d, capture_output=True, text=True)
        assert r.returncode == 0 and int(r.stdout.strip()) > 10, r.stderr


def test_sampler():
    logits = torch.tensor([0.0, 5.0, 1.0, 4.9])
    assert ch.sample_next(logits, 0.0, 0, 0.0) == 1
    g = torch.Generator().manual_seed(0)
    draws = {ch.sample_next(logits, 1.0, 2, 0.0, g) for _ in range(200)}
    assert draws == {1, 3}
    draws = {ch.sample_next(logits, 1.0, 0, 0.5, g) for _ in range(200)}
    assert draws <= {1, 3} and 1 in draws
    assert {ch.sample_next(logits, 1.0, 0, 1e-6, g) for _ in range(20)} == {1}


def test_stream_renderer_dims_think_and_buffers_tool_calls():
    buf = io.StringIO()
    r = ch.StreamRenderer(buf)
    full = 'hi <think>plan</think>ok <tool_call>{"name": "f"}</tool_call> done'
    for i in range(1, len(full) + 1, 3):
        r.feed(full[:i])
    r.feed(full)
    r.flush()
    out = buf.getvalue()
    assert "<think>" not in out and "<tool_call>" not in out
    assert "tool_call: {\"name\": \"f\"}" in out and out.startswith("hi ") and out.rstrip().endswith("done")


def test_chat_session_generates_and_applies_settings(packed):
    d, tok, cfg, model = packed
    out = str(d / "chat.aio")
    pk.build_package(str(d / "m.pt"), str(d / "tok.json"), os.path.join(ROOT, "chat_template.jinja"), out, "none")
    s = ch.Settings(device="cpu", dtype="fp32", temperature=0.0, top_k=0, top_p=0.9, max_new=6, window=0, alpha=0.05, beta=0.1)
    sess = ch.ChatSession(out, s)
    assert s.window == 16 and abs(s.alpha - cfg.tria_carrier_alpha) < 1e-12
    msgs = [{"role": "user", "content": "alpha beta"}]
    buf = io.StringIO()
    reply, interrupted = sess.generate_turn(msgs, out=buf)
    assert reply["role"] == "assistant" and not interrupted
    # greedy engine output equals the model's own token-by-token step path
    ids = sess.chat.render_prompt_ids(msgs)
    st, lg = None, None
    with torch.no_grad():
        for p, t in enumerate(ids):
            lg, st = sess.model.step(torch.tensor([t]), p, st)
        want = []
        for i in range(6):
            n = int(lg[0].argmax())
            if n in sess.chat.stop_ids:
                break
            want.append(n)
            lg, st = sess.model.step(torch.tensor([n]), len(ids) + i, st)
    assert reply["content"] == tok.decode(want, skip_special_tokens=True) or reply.get("tool_calls")
    assert sess.set("beta", "1.5") is not None and sess.set("alpha", "-1") is not None and sess.set("window", "0") is not None
    assert sess.set("window", "8") is None and sess.cfg.tria_temporal_window == 8
    assert sess.set("beta", "0.2") is None and sess.cfg.tria_polarm_beta == 0.2
    assert sess.set("dtype", "int8") is not None and sess.set("top_k", "x") == "couldn't parse 'x' for top_k"
    assert sess.set("device", "cuda:0") is not None or torch.cuda.is_available()
    handled, leave = ch.handle_command("/reset", sess, msgs)
    assert handled and not leave and msgs == []
    assert ch.handle_command("/system be brief", sess, msgs) == (True, False) and msgs[0]["role"] == "system"
    assert ch.handle_command("/ex", sess, msgs) == (True, True)
    assert ch.handle_command("/temperature 0.3", sess, msgs) == (True, False) and s.temperature == 0.3
    assert ch.handle_command("hello", sess, msgs) == (False, False)
    with pytest.raises(ValueError):
        ch.load_aio(str(d / "m.pt"), torch.device("cpu"))


def _fake_llama(d, hidden_size=32, heads=4, kv=2, inter=86, layers=2, vocab=64):
    import json as js
    from loomformer_paraplex_b200.tools import cloner as cl
    os.makedirs(d, exist_ok=True)
    js.dump({"architectures": ["LlamaForCausalLM"], "hidden_size": hidden_size, "num_attention_heads": heads,
             "num_key_value_heads": kv, "num_hidden_layers": layers, "vocab_size": vocab, "rope_theta": 10000.0,
             "max_position_embeddings": 64, "tie_word_embeddings": True, "intermediate_size": inter,
             "_name_or_path": "tiny/llama"}, open(os.path.join(d, "config.json"), "w"))
    g = torch.Generator().manual_seed(0)
    hd = hidden_size // heads
    T = {"model.embed_tokens.weight": torch.randn(vocab, hidden_size, generator=g).bfloat16(),
         "model.norm.weight": torch.ones(hidden_size).bfloat16()}
    for i in range(layers):
        p = f"model.layers.{i}."
        T[p + "input_layernorm.weight"] = torch.rand(hidden_size, generator=g).bfloat16()
        T[p + "post_attention_layernorm.weight"] = torch.rand(hidden_size, generator=g).bfloat16()
        T[p + "self_attn.q_proj.weight"] = torch.randn(heads * hd, hidden_size, generator=g).bfloat16()
        T[p + "self_attn.k_proj.weight"] = torch.randn(kv * hd, hidden_size, generator=g).bfloat16()
        T[p + "self_attn.v_proj.weight"] = torch.randn(kv * hd, hidden_size, generator=g).bfloat16()
        T[p + "self_attn.o_proj.weight"] = torch.randn(hidden_size, heads * hd, generator=g).bfloat16()
        T[p + "mlp.up_proj.weight"] = torch.randn(inter, hidden_size, generator=g).bfloat16()
        T[p + "mlp.gate_proj.weight"] = torch.randn(inter, hidden_size, generator=g).bfloat16()
        T[p + "mlp.down_proj.weight"] = torch.randn(hidden_size, inter, generator=g).bfloat16()
    cl.write_safetensors(os.path.join(d, "model.safetensors"), T)
    return T


def test_cloner_scan_and_clone(tmp_path):
    from loomformer_paraplex_b200.tools import cloner as cl
    from loomformer_paraplex_b200.train.engine import train_lr_overrides
    donor_dir = str(tmp_path / "donor")
    T = _fake_llama(donor_dir)
    from safetensors.torch import load_file            # the file written by the minimal writer is standard
    assert torch.equal(load_file(os.path.join(donor_dir, "model.safetensors"))["model.norm.weight"], T["model.norm.weight"])
    back = cl.read_safetensors(os.path.join(donor_dir, "model.safetensors"))
    assert all(torch.equal(back[k], T[k]) for k in T)
    env = dict(os.environ, PYTHONPATH=ROOT)
    tool = os.path.join(ROOT, "loomcloner.py")
    y = str(tmp_path / "clone.yaml")
    r = subprocess.run([sys.executable, tool, "--scan", donor_dir, "--out", y, "--steps", "90", "--lr", "1e-4",
                        "--paraplex-gate-proj", "--final-norm"], env=env, capture_output=True, text=True)
    assert r.returncode == 0 and "mapping=llama" in r.stdout, r.stderr
    cfg = Config.from_yaml(y)
    assert (cfg.model_dim, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.layers, cfg.vocab) == (32, 4, 2, 8, 2, 64)
    assert cfg.hidden == 88 and cfg.warmup_steps == 3 and cfg.optimizer == "atom" and cfg.cloned and cfg.cloned_from == "tiny/llama"
    assert cfg.paraplex_gate_proj and cfg.final_norm and cfg.tied_embeddings
    byname = {e["name"]: e for e in cfg.train_lr}
    assert abs(byname["attn.qkv_weight"]["lr"] - 1e-5) < 1e-12 and abs(byname["ln_ffn.bias"]["lr"] - 1e-4) < 1e-12
    assert "not divisible by n_q_heads=4" in open(y).read()
    out = str(tmp_path / "clone.pt")
    r = subprocess.run([sys.executable, tool, "--clone", y, "--donor", donor_dir, "--out", out], env=env,
                       capture_output=True, text=True)
    assert r.returncode == 0 and "saved ->" in r.stdout, r.stdout + r.stderr
    blob = torch.load(out, weights_only=True)
    st = blob["model"]
    assert blob["cloned"] and blob["step"] == 0 and st["emb.weight"].dtype == torch.bfloat16
    assert torch.equal(st["blocks.1.attn.qkv_weight"], torch.cat([T["model.layers.1.self_attn.q_proj.weight"],
                       T["model.layers.1.self_attn.k_proj.weight"], T["model.layers.1.self_attn.v_proj.weight"]], 0))
    assert torch.equal(st["blocks.0.ffn.w1_real.weight"][:86], T["model.layers.0.mlp.up_proj.weight"])
    assert float(st["blocks.0.ffn.w1_real.weight"][86:].abs().sum()) == 0.0
    assert torch.equal(st["blocks.0.ffn.w2.weight"][:, :86], T["model.layers.0.mlp.down_proj.weight"])
    assert torch.equal(st["blocks.0.ffn.gate_proj.weight"][:86], T["model.layers.0.mlp.gate_proj.weight"])
    assert torch.equal(st["ln_final.weight"], T["model.norm.weight"]) and torch.equal(st["emb.weight"], T["model.embed_tokens.weight"])
    assert yaml_resume(y) == out
    # the generated overrides bind to real parameter names
    cfg2 = Config.from_yaml(y)
    model = Model(cfg2)
    mults = train_lr_overrides(model, cfg2)
    assert abs(mults["blocks.0.attn.qkv_weight"] - 0.1) < 1e-9 and abs(mults["blocks.1.ln_attn.bias"] - 1.0) < 1e-9


def yaml_resume(path):
    import yaml
    return yaml.safe_load(open(path))["resume"]


def test_every_shipped_config_loads_and_resolves():
    from loomformer_paraplex_b200.config import resolve
    names = sorted(os.listdir(os.path.join(ROOT, "cfg")))
    assert {"alt.yaml", "alt2.yaml", "chk.yaml", "chk_sft.yaml", "mini.yaml", "nano.yaml", "nano_chk.yaml", "nano_sft.yaml",
            "sft.yaml", "smol360.yaml"} <= set(names)
    for n in names:
        cfg = Config.from_yaml(os.path.join(ROOT, "cfg", n))
        d = resolve(cfg, calibrate=False)
        assert d.n == d.qh * d.hd and d.hidden % d.qh == 0, n
    nano = resolve(Config.from_yaml(os.path.join(ROOT, "cfg", "nano.yaml")), calibrate=False)
    assert (nano.n, nano.qh, nano.kvh, nano.hd, nano.hidden, nano.layers) == (768, 8, 2, 96, 3072, 10)


def test_replica_pool_serves_in_order_and_detects_a_dead_replica(packed):
    """Two CPU replicas give what a single engine gives; a replica that dies is reported instead of waited for."""
    from loomformer_paraplex_b200.serve.decode import DecodeEngine
    from loomformer_paraplex_b200.serve.replicas import ReplicaPool
    from loomformer_paraplex_b200.serve.runtime import load_model
    d, tok, cfg, _ = packed
    path = str(d / "m.pt")
    prompts = [[(7 * i + j) % tok.vocab_size for j in range(12)] for i in range(5)]
    model, *_ = load_model(path, torch.device("cpu"), tokenizer=tok)
    eng = DecodeEngine(model, batch=2, use_graph=False)
    want = []
    for lo in range(0, 5, 2):
        rows = torch.tensor(prompts[lo:lo + 2])
        n = rows.shape[0]
        if n < 2:
            rows = torch.cat((rows, rows[:1]), 0)
        want += eng.generate(rows, 4)[:n].tolist()
    with ReplicaPool(path, ["cpu", "cpu"], batch=2) as pool:
        got = pool.generate(prompts, 4)
        assert got == want
        pool.procs[0].terminate(); pool.procs[0].join()
        with pytest.raises(RuntimeError):
            pool.generate(prompts[:4], 2, timeout=3.0)
    with pytest.raises(RuntimeError):
        ReplicaPool(str(d / "missing.pt"), ["cpu"], batch=1, start_timeout=60)


def test_export_package_reproduces_the_forward(tmp_path):
    """`--export-aoti` route: the saved program (AOTInductor package or ExportedProgram) runs without model code."""
    from loomformer_paraplex_b200.serve.runtime import export_package
    cfg = Config(vocab=256, seq_len=32, model_dim=32, n_q_heads=4, n_kv_heads=2, hidden=64, layers=2, activation="pvpowlu",
                 tria_carry_enabled=True, tria_temporal_auto=False, tria_temporal_window=16)
    torch.manual_seed(0)
    model = Model(cfg).eval()
    ckpt.save_checkpoint(str(tmp_path / "e.pt"), cfg, model, None, "adamw", 0, 0)
    path = export_package(str(tmp_path / "e.pt"), str(tmp_path / "e.pt2"), torch.device("cpu"))
    x = torch.randint(0, 256, (1, 32))
    with torch.no_grad():
        want = model(x)
    try:
        got = torch.export.load(path).module()(x)
    except Exception:
        got = torch._inductor.aoti_load_package(path)(x)
    assert torch.allclose(got, want, atol=1e-4)
