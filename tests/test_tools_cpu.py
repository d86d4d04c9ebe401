"""Command-line tools and utilities on the CPU: fp8 -> bf16 checkpoint conversion, the generate
CLI (single and bench modes, child process), integer quantisation definitions, debug / profiling
helpers (the reference's tests/funcs/print.py exercises its tensor print the same way)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fp8_cast_bf16_roundtrip(tmp_path):
    from safetensors.torch import load_file, save_file
    from gvirt_b200.ops import reference as ref
    from gvirt_b200.tools.fp8_cast_bf16 import convert, dequant_block128
    src, dst = tmp_path / "fp8", tmp_path / "bf16"
    src.mkdir()
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(256, 384, generator=g) * 0.1
    w2 = torch.randn(200, 130, generator=g) * 0.1          # not multiples of 128
    norm = torch.ones(384, dtype=torch.bfloat16)
    q1, s1 = ref.quant_fp8_block(w1)
    q2, s2 = ref.quant_fp8_block(w2)
    save_file({"a.weight": q1, "n.weight": norm, "b.weight_scale_inv": s2}, str(src / "model-00001-of-00002.safetensors"))
    save_file({"b.weight": q2, "a.weight_scale_inv": s1}, str(src / "model-00002-of-00002.safetensors"))
    index = {"metadata": {}, "weight_map": {"a.weight": "model-00001-of-00002.safetensors",
                                             "n.weight": "model-00001-of-00002.safetensors",
                                             "b.weight_scale_inv": "model-00001-of-00002.safetensors",
                                             "b.weight": "model-00002-of-00002.safetensors",
                                             "a.weight_scale_inv": "model-00002-of-00002.safetensors"}}
    (src / "model.safetensors.index.json").write_text(json.dumps(index))
    (src / "config.json").write_text(json.dumps({"hidden_size": 384, "quantization_config": {"quant_method": "fp8"}}))
    (src / "tokenizer.json").write_text("{}")
    stats = convert(str(src), str(dst), "cpu")
    assert stats["converted"] == 2 and stats["dropped_scales"] == 2 and not stats["missing_scale"]
    out = {}
    for f in sorted(dst.glob("*.safetensors")):
        out.update(load_file(str(f)))
    assert set(out) == {"a.weight", "b.weight", "n.weight"}
    assert out["a.weight"].dtype == torch.bfloat16 and out["b.weight"].shape == (200, 130)
    assert torch.equal(out["a.weight"], dequant_block128(q1, s1))
    assert (out["a.weight"].float() - w1).abs().max() < 0.02 and (out["b.weight"].float() - w2).abs().max() < 0.02
    new_index = json.loads((dst / "model.safetensors.index.json").read_text())
    assert set(new_index["weight_map"]) == {"a.weight", "b.weight", "n.weight"}
    cfg = json.loads((dst / "config.json").read_text())
    assert "quantization_config" not in cfg and cfg["torch_dtype"] == "bfloat16"
    assert (dst / "tokenizer.json").exists()


def _cli(*args):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run([sys.executable, "-m", "gvirt_b200.tools.generate", *args], capture_output=True, text=True,
                       cwd=ROOT, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    return r.stdout


def test_generate_cli_single_and_bench():
    out = _cli("--preset", "tiny-qwen2", "--device", "cpu", "--prompt-ids", "1,2,3,4", "--prompt-ids", "7,8",
               "--max-tokens", "6", "--json")
    rows = [json.loads(l) for l in out.splitlines() if l.startswith("{")]
    assert [r["prompt_ids"] for r in rows] == [[1, 2, 3, 4], [7, 8]] and all(len(r["output_ids"]) == 6 for r in rows)
    out2 = _cli("--preset", "tiny-qwen2", "--device", "cpu", "--prompt-ids", "1,2,3,4", "--max-tokens", "6", "--json")
    assert json.loads(out2.splitlines()[0])["output_ids"] == rows[0]["output_ids"]   # batch-invariant greedy
    b = _cli("--preset", "tiny-qwen2", "--device", "cpu", "--mode", "bench", "--batch", "2", "--prompt-len", "24",
             "--max-tokens", "8", "--iters", "2", "--json")
    rec = json.loads([l for l in b.splitlines() if l.startswith("{")][-1])
    assert rec["mode"] == "bench" and rec["decode_tok_s"] > 0 and rec["prefill_tok_s"] > 0


def test_int_quant_definitions():
    from gvirt_b200.ops import quant_ops as Q
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 64, generator=g).bfloat16()
    q, s = Q.quant_i8_dynamic(x)
    assert q.dtype == torch.int8 and q.abs().max() <= 127
    assert torch.allclose(q.float() * s[:, None], x.float(), atol=float(s.max()) * 0.51 + 1e-3)
    w = torch.randn(16, 64, generator=g) * 0.1
    ws = w.abs().amax(-1) / 127
    wq = torch.clamp(torch.round(w / ws[:, None]), -128, 127).to(torch.int8)
    y = Q.linear_w8a8(x, wq, ws, out=torch.empty(9, 16))
    assert (y - x.float() @ w.t()).abs().max() < 0.08
    packed = torch.tensor([[0x8F, 0x70]], dtype=torch.uint8)      # nibbles (low first): -1, -8, 0, 7
    assert Q.unpack_i4(packed).tolist() == [[-1, -8, 0, 7]]
    zero = torch.zeros(2, 64, dtype=torch.bfloat16)
    qz, sz = Q.quant_i8_dynamic(zero)
    assert int(qz.abs().max()) == 0 and float(sz.max()) == 0.0       # all-zero rows do not divide by zero


def test_debug_and_profiling_helpers(capfd):
    from gvirt_b200.utils import debug, profiling
    debug.configure(3, "forward")
    assert debug.enabled("forward") and not debug.enabled("comm")
    for shape in [(5,), (3, 4), (2, 3, 4)]:                          # 1-D / 2-D / 3-D like the reference's print test
        t = torch.arange(int(torch.tensor(shape).prod()), dtype=torch.float32).reshape(shape)
        text = debug.describe("t", t)
        assert f"shape={shape}" in text and "nan=0" in text
    debug.log("forward", "hello from the test")
    debug.log("comm", "must not appear")
    out = capfd.readouterr()
    assert "(R3)" in (out.out + out.err) and "hello from the test" in (out.out + out.err)
    assert "must not appear" not in (out.out + out.err)
    with pytest.raises(FloatingPointError):
        debug.check_nan_inf("bad", torch.tensor([1.0, float("inf")]))
    debug.configure(0, "")
    # layer diff between two runs of the tiny model: identical weights -> no divergence; perturbed -> found
    from gvirt_b200.engine.llm import LLM
    from gvirt_b200.engine.scheduler import SamplingParams
    from gvirt_b200.models import presets
    cfg = presets.get("tiny-qwen2", max_batch_size=2)
    a = LLM.from_config(cfg, seed=0, device="cpu")
    b = LLM.from_config(presets.get("tiny-qwen2", max_batch_size=2), seed=0, device="cpu")
    d = debug.LayerDiff()
    sp = SamplingParams(max_tokens=1, ignore_eos=True)
    with d.record("a", a.model):
        a.generate([[1, 2, 3]], sp)
    with d.record("b", b.model):
        b.generate([[1, 2, 3]], sp)
    assert "all records agree" in d.report("a", "b")
    b.model.w.layers[1].w_o.mul_(1.5)
    with d.record("b2", b.model):
        b.generate([[1, 2, 3]], sp)
    rep = d.report("a", "b2")
    assert "first divergence at record" in rep and "DIFF" in rep
    with debug.paranoid(a.model):
        a.generate([[4, 5]], sp)
    with profiling.OpTable() as ops:
        a.generate([[4, 5, 6]], sp)
    assert ops.totals() == {} or all(c > 0 for c, _ in ops.totals().values())   # CPU path makes no native calls
    with profiling.DeviceTimer() as t:
        sum(range(10000))
    assert t.ms > 0 and t.max_ms() == t.ms
    assert profiling.time_fn(lambda: None, warmup=1, iters=3) >= 0


def test_cpu_affinity_helpers(tmp_path):
    from gvirt_b200.utils import affinity as A
    assert A.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert A.parse_cpulist("") == []
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:3b:00.0"
    dev.mkdir(parents=True)
    (dev / "local_cpulist").write_text("0-15,64-79\n")
    cpus = A.gpu_local_cpus("00000000:3B:00.0", str(tmp_path))
    assert cpus == list(range(16)) + list(range(64, 80))
    assert A.gpu_local_cpus("0000:ff:00.0", str(tmp_path)) is None
    assert A.split_for_rank(cpus, 1, 4) == [8, 9, 10, 11, 12, 13, 14, 15]
    assert A.split_for_rank([0, 1], 3, 4) == [0, 1]
    assert A.bind_to_gpu(0) is None or isinstance(A.bind_to_gpu(0), list)     # no GPU here: a no-op
    assert A.bind_rank(0) is None or isinstance(A.bind_rank(0), list)
    from gvirt_b200.config import EnvFlags
    assert EnvFlags.from_env({"GVIRT_CPU_BINDING": "1"}).cpu_binding and not EnvFlags.from_env({}).cpu_binding


def test_comm_sizing_rules(monkeypatch):
    """Heap sizing and the MoE exchange capacity rule (worst case, ratio, scratch budget, floor)."""
    from gvirt_b200 import config as gcfg
    from gvirt_b200.models import presets
    from gvirt_b200.parallel.moe_a2a import a2a_capacity
    from gvirt_b200.parallel.setup import a2a_bytes, heap_bytes
    ds = presets.get("deepseek-v3", ep_size=8)
    worst = 8 * 2048
    expect = 8 * 2048 * 8 / 256
    cap = a2a_capacity(ds, 8, 2048)
    assert 4 * expect <= cap <= worst
    monkeypatch.setenv("GVIRT_A2A_SCRATCH_GB", "1000")
    gcfg.reload_flags()
    assert a2a_capacity(ds, 8, 2048) == worst                       # no budget pressure: worst case
    monkeypatch.setenv("GVIRT_ACTIVE_TOKENS_RATIO_PER_EP", "0.1")
    gcfg.reload_flags()
    assert a2a_capacity(ds, 8, 2048) == max(int(4 * expect), int(0.1 * worst))
    monkeypatch.setenv("GVIRT_A2A_SCRATCH_GB", "0.001")
    gcfg.reload_flags()
    assert a2a_capacity(ds, 8, 2048) == int(4 * expect)             # never below four times the expected load
    monkeypatch.delenv("GVIRT_A2A_SCRATCH_GB")
    monkeypatch.delenv("GVIRT_ACTIVE_TOKENS_RATIO_PER_EP")
    gcfg.reload_flags()
    assert a2a_bytes(ds, 8, 2048) > a2a_capacity(ds, 8, 2048) * 32 * ds.hidden_size
    ll = presets.get("llama-3-8b", tp_size=8, max_num_batched_tokens=8192)
    assert heap_bytes(ll, 8) >= 4 * 2 * 9 * 128 * 4096 * 4          # the fused all-reduce regions fit
    assert heap_bytes(presets.get("llama-3-8b", tp_size=2, max_num_batched_tokens=8192), 2) >= 1 << 30


def test_runtime_stub_is_current_and_parses():
    """The committed .pyi of the C++ runtime module matches what the bindings export."""
    import ast
    from pathlib import Path
    from gvirt_b200.tools import gen_stubs
    assert gen_stubs.main(["--check"]) == 0
    stub = Path(gen_stubs.__file__).resolve().parent.parent / "lib" / "_gvirt_runtime.pyi"
    tree = ast.parse(stub.read_text())
    classes = {n.name for n in tree.body if isinstance(n, ast.ClassDef)}
    assert {"TensorPool", "BlockManager", "CoreAssigner", "NgramIndex", "Sock"} <= classes


def test_persistent_gemm_tile_walk_covers_every_tile_once():
    """Index arithmetic of gemm_persist.cu's tile walk, through its host-side entry point."""
    import ctypes
    from gvirt_b200 import _native
    f = _native.kernels().gv_gemm_persistent_tile
    f.argtypes = [ctypes.c_longlong] * 3 + [ctypes.POINTER(ctypes.c_int)] * 2
    for tm, tn in ((64, 24), (1, 1), (17, 3), (16, 16), (33, 1), (9, 112)):
        seen = set()
        for t in range(tm * tn):
            p, q = ctypes.c_int(), ctypes.c_int()
            assert f(t, tm, tn, ctypes.byref(p), ctypes.byref(q)) == 0
            assert p.value % 128 == 0 and q.value % 256 == 0
            seen.add((p.value // 128, q.value // 256))
        assert seen == {(i, j) for i in range(tm) for j in range(tn)}
    p, q = ctypes.c_int(), ctypes.c_int()
    assert f(6, 2, 3, ctypes.byref(p), ctypes.byref(q)) != 0      # out of range


def test_peer_memory_paths_stay_inside_a_node():
    """The symmetric heap (peer-mapped memory) is only built for groups whose ranks share a node;
    16 ranks on two nodes: TP8 groups qualify, the EP16 group does not."""
    from gvirt_b200.parallel.state import ParallelContext
    from gvirt_b200.parallel.symm import group_is_single_node
    assert group_is_single_node(range(8), 8) and group_is_single_node([8, 9, 10, 11], 8)
    assert not group_is_single_node([7, 8], 8) and not group_is_single_node(range(16), 8)
    ctx = ParallelContext(world=16, rank=9, tp=8, dp=2, ep=16, moe_tp=1)
    assert group_is_single_node(ctx.tp_ranks(), 8) and not group_is_single_node(ctx.ep_ranks(), 8)
    assert group_is_single_node(ctx.ep_ranks(), 16)          # one 16-GPU node


def test_paranoid_mode_from_the_environment(monkeypatch):
    """GVIRT_PARANOID=1: every layer output is checked as it is produced; a NaN planted in a
    weight is reported with the layer it first shows up in, a healthy model runs as usual."""
    import pytest
    import torch
    from gvirt_b200 import config as gcfg
    from gvirt_b200.engine.llm import LLM
    from gvirt_b200.engine.scheduler import SamplingParams
    from gvirt_b200.models import presets
    monkeypatch.setenv("GVIRT_PARANOID", "1")
    gcfg.reload_flags()
    try:
        llm = LLM.from_config(presets.get("tiny-qwen2"), seed=0, device="cpu")
        assert llm.paranoid and llm.model.debug_hook is not None
        out = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=3, ignore_eos=True))[0].output
        assert len(out) == 3
        llm.model.w.layers[1].w_down[0, 0] = float("nan")
        with pytest.raises(Exception) as ei:
            llm.generate([[4, 5, 6]], SamplingParams(max_tokens=2, ignore_eos=True))
        assert "layer 1" in str(ei.value)
    finally:
        monkeypatch.delenv("GVIRT_PARANOID")
        gcfg.reload_flags()


def test_rendezvous_from_runtime_variables_without_torchrun(tmp_path):
    """Two processes started by hand (RANK / WORLD_SIZE only): the rendezvous address and port
    come from GVIRT_NODE_IPS / GVIRT_PORT."""
    import os
    import socket
    import subprocess
    import sys
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    code = "\n".join([
        "import os, torch, torch.distributed as dist",
        "from gvirt_b200.parallel import state",
        "ctx = state.init_parallel(tp=2, backend='gloo', device='cpu', timeout_s=60)",
        "t = torch.tensor([ctx.rank + 1.0]); dist.all_reduce(t)",
        "assert t.item() == 3.0 and os.environ['MASTER_ADDR'] == '127.0.0.1'",
        "print('RDV_OK', ctx.rank)"])
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = {k: v for k, v in os.environ.items() if k not in ("MASTER_ADDR", "MASTER_PORT")}
        env.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2", GVIRT_NODE_IPS="127.0.0.1,127.0.0.2",
                   GVIRT_PORT=str(port), PYTHONPATH=root)
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True, cwd=root))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert all("RDV_OK" in o for o in outs)


def test_debug_forward_category_prints_layer_summaries(monkeypatch, capfd):
    """GVIRT_DEBUG_ON=forward: the engine prints tensor summaries of layer 0 (and the first MoE
    layer) at its three probe points; other layers and other categories stay quiet."""
    from gvirt_b200 import config as gcfg
    from gvirt_b200.engine.llm import LLM
    from gvirt_b200.engine.scheduler import SamplingParams
    from gvirt_b200.models import presets
    from gvirt_b200.utils import debug as dbg
    monkeypatch.setenv("GVIRT_DEBUG_ON", "forward")
    gcfg.reload_flags()
    try:
        llm = LLM.from_config(presets.get("tiny-qwen2"), seed=0, device="cpu")
        llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True))
        out = capfd.readouterr()
        text = out.out + out.err
        assert "L0 in" in text and "L0 after_attn" in text and "L0 after_ffn" in text
        assert "L1 in" not in text and "shape=(3, 256)" in text
    finally:
        monkeypatch.delenv("GVIRT_DEBUG_ON")
        gcfg.reload_flags()
        dbg.configure(rank=0)
    quiet = LLM.from_config(presets.get("tiny-qwen2"), seed=0, device="cpu")
    quiet.generate([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True))
    out = capfd.readouterr()
    assert "L0 in" not in out.out + out.err


def test_op_checks_compare_every_op_with_its_definition(monkeypatch):
    """The wrapper copies arguments before the call, runs the definition on the copies and
    compares results and in-place updates; a wrong kernel is named with its argument."""
    import torch
    from gvirt_b200.ops import functional as F
    from gvirt_b200.utils import op_checks as oc
    oc.reset_stats()
    n = oc.enable(force=True)
    try:
        assert n > 30 and hasattr(F.linear, "_gv_unchecked") and not hasattr(F.interleave_gate_up, "_gv_unchecked")
        assert oc.enable(force=True) == 0                       # idempotent
        x, w = torch.randn(5, 16), torch.randn(8, 16)
        res = torch.zeros(5, 16)
        y = F.add_rmsnorm(x, res, torch.ones(16), 1e-6)        # updates `res` in place; calls F.norm inside
        assert torch.allclose(res, x) and y.shape == (5, 16)
        assert oc.stats.per_op == {"functional.add_rmsnorm": 1}   # the inner op is covered by the outer check
        F.linear(x, w)
        assert oc.stats.checked == 2 and not oc.stats.mismatches
        # a whole engine run goes through the wrappers
        from gvirt_b200.engine.llm import LLM
        from gvirt_b200.engine.scheduler import SamplingParams
        from gvirt_b200.models import presets
        llm = LLM.from_config(presets.get("tiny-qwen2"), seed=0, device="cpu")
        llm.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=3, ignore_eos=True))
        assert oc.stats.checked > 20 and not oc.stats.mismatches
        assert any(k.startswith("functional.paged_attention") for k in oc.stats.per_op)
        # sampling with a temperature is random by design: counted, not compared
        llm.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=2, temperature=0.8, ignore_eos=True))
        assert oc.stats.skipped_random > 0
        # arguments over the size limit are not copied
        oc._cfg["max_bytes"] = 16
        before = oc.stats.skipped_large
        F.linear(x, w)
        assert oc.stats.skipped_large == before + 1
        oc._cfg["max_bytes"] = 512 << 20
    finally:
        oc.disable()
    assert not hasattr(F.linear, "_gv_unchecked")

    # a kernel that is wrong in its output, and one that forgets its in-place update
    def definition(x, w, out):
        out.copy_(x @ w.t())
        return out

    def wrong_value(x, w, out):
        out.copy_(x @ w.t() + 0.5)
        return out

    def forgets_out(x, w, out):
        return x @ w.t()

    oc._cfg["force"] = True
    try:
        x, w = torch.randn(4, 8), torch.randn(3, 8)
        oc.checked(definition, "toy.linear", definition)(x, w, out=torch.zeros(4, 3))
        import pytest
        with pytest.raises(oc.OpMismatch, match=r"toy.linear: result is off by"):
            oc.checked(wrong_value, "toy.linear", definition)(x, w, out=torch.zeros(4, 3))
        with pytest.raises(oc.OpMismatch, match=r"toy.linear: kw\['out'\] is off by"):
            oc.checked(forgets_out, "toy.linear", definition)(x, w, out=torch.zeros(4, 3))
        oc._cfg["on_mismatch"] = "log"
        oc.reset_stats()
        oc.checked(wrong_value, "toy.linear", definition)(x, w, out=torch.zeros(4, 3))
        assert len(oc.stats.mismatches) == 2          # the result and the out= tensor
        ids = torch.arange(100)
        assert oc.compare("t", "ids", ids, ids.clone()) is None
        flipped = ids.clone()
        flipped[:2] += 1
        assert oc.compare("t", "ids", flipped, ids) is None                  # 2 % differ: ties
        flipped[:10] += 1
        assert "10.0 %" in oc.compare("t", "ids", flipped, ids)
        assert "shape" in oc.compare("t", "x", torch.zeros(2, 3), torch.zeros(3, 2))
        assert "NaN" in oc.compare("t", "x", torch.tensor([float("nan")]), torch.tensor([1.0]))
    finally:
        oc._cfg["on_mismatch"] = "raise"
        oc._cfg["force"] = False


def test_gemm_sweep_outlier_filter_decision_and_report(tmp_path, capsys):
    import json
    from gvirt_b200.tools import gemm_sweep as gs
    assert gs.robust_mean([10.0, 10.2, 9.9, 10.1, 55.0]) == sum([10.0, 10.2, 9.9, 10.1]) / 4     # the spike is dropped
    assert gs.robust_mean([10.0, 30.0]) == 20.0                                                   # too few to judge
    assert gs.decide({0: 10.0, 1: 10.0, 2: 9.8, 4: 9.0}, 0.03) == (4, True)
    assert gs.decide({0: 10.0, 1: 10.2, 2: 9.8}, 0.03) == (2, False)                              # inside the margin
    raw = {"preset": "p", "tp": 1, "shapes": [
        {"shape": "qkv", "M": 64, "N": 6144, "K": 4096, "samples": {"0": [10, 10, 10], "1": [11, 11, 11], "2": [9, 9, 9.3]}},
        {"shape": "down", "M": 64, "N": 4096, "K": 14336, "samples": {"0": [20, 20, 20, 20, 90], "4": [19.9, 20, 20, 20.1]}}]}
    (tmp_path / "raw.json").write_text(json.dumps(raw))
    assert gs.main(["--report", str(tmp_path / "raw.json")]) == 0
    out = capsys.readouterr().out.splitlines()
    assert out[0].startswith("| shape | M | N | K | auto | x1 | x2 | x4 | best | override |")
    assert out[2] == "| qkv | 64 | 6144 | 4096 | 10.00 | 11.00 | 9.10 | - | x2 | yes |"
    assert out[3] == "| down | 64 | 4096 | 14336 | 20.00 | - | - | 20.00 | x4 | no |"


def test_causal_softmax_definition_matches_softmax_over_padded_rows():
    """Row m is a softmax over its first calc_len + m entries (the reference's own check pads the
    row with -inf and compares with torch.softmax, xlite/tests/kernels/softmax.py); an empty row
    gives zeros, and the op works in place."""
    import torch

    from gvirt_b200.ops import functional as F
    from gvirt_b200.ops import reference as ref
    g = torch.Generator().manual_seed(0)
    for rows, cols, calc in [(1, 128, 3), (4, 128, 78), (3, 1152, 1035), (2, 64, 64), (2, 64, 200)]:
        x = torch.randn(rows, cols, generator=g)
        padded = x.clone()
        for m in range(rows):
            padded[m, calc + m:] = float("-inf")
        want = torch.softmax(padded, dim=-1)
        assert torch.allclose(ref.causal_softmax(x, calc), want, atol=1e-6)
        y = x.clone()
        assert F.softmax(y, calc) is y and torch.allclose(y, want, atol=1e-6)
        assert torch.allclose(y.sum(-1), torch.ones(rows), atol=1e-5)
    z = torch.full((2, 16), float("-inf"))
    assert torch.equal(ref.causal_softmax(z, 4), torch.zeros(2, 16))
    assert torch.equal(ref.causal_softmax(torch.randn(1, 16), 0), torch.zeros(1, 16))
    meta = torch.empty(2, 16, device="meta")
    assert F.softmax(meta, 3) is meta


def test_moe_exchange_step_size_keeps_the_exchange_exact(monkeypatch):
    """With the default ratio the fused MoE exchange never drops a row: where the slot-addressed
    scratch cannot hold the worst case of a full step, the step shrinks instead; a ratio below 1
    (the approximate mode) leaves the step alone; a decode batch that cannot fit is an error."""
    import pytest
    from gvirt_b200 import config
    from gvirt_b200.models import presets
    from gvirt_b200.parallel.moe_a2a import a2a_capacity, a2a_exact_tokens
    from gvirt_b200.parallel.setup import fit_step_to_exchange
    kw = dict(ep_size=8, dp_size=8, tp_size=1, max_batch_size=32, max_num_batched_tokens=8192)
    cfg = presets.get("deepseek-v3", **kw)
    R = 8
    assert a2a_capacity(cfg, R, 8192) < R * 8192               # memory cuts the capacity
    step = fit_step_to_exchange(cfg, R)
    assert step == cfg.max_num_batched_tokens < 8192 and step % 128 == 0
    assert R * step <= a2a_capacity(cfg, R, step)              # worst case of the new step fits
    assert a2a_exact_tokens(cfg, R, step) == step
    small = presets.get("qwen3-30b-a3b", **kw)
    assert fit_step_to_exchange(small, R) == 8192              # fits as it is
    monkeypatch.setenv("GVIRT_ACTIVE_TOKENS_RATIO_PER_EP", "0.25")
    config.reload_flags()
    try:
        cfg2 = presets.get("deepseek-v3", **kw)
        assert fit_step_to_exchange(cfg2, R) == 8192           # approximate mode: untouched
    finally:
        monkeypatch.delenv("GVIRT_ACTIVE_TOKENS_RATIO_PER_EP")
        config.reload_flags()
    # a decode batch larger than what fits exactly is refused with a clear message
    import gvirt_b200.parallel.moe_a2a as A
    monkeypatch.setattr(A, "a2a_capacity", lambda cfg, R, cap: 64 * R)
    with pytest.raises(ValueError, match="decode step"):
        fit_step_to_exchange(presets.get("deepseek-v3", **dict(kw, max_batch_size=256)), R)
