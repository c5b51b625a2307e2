"""Developer tools: log comparison."""
import pytest
from pathlib import Path

ROOT_DIR = Path(__file__).resolve().parents[1]
from pithtrain_b200.tools.validate_correctness import compare

LINE = ("[2026-01-01 00:00:0{i}] step 0000000{i}/00000025 | step-time {t} sec | cross-entropy-loss {ce} | "
        "load-balance-loss 1.02e-03 | tokens-per-second 15,942 | peak-gpu-memory 142.13 GB\n")


def _write(path, ces, t="8.2"):
    path.write_text("noise\n" + "".join(LINE.format(i=i + 1, t=t, ce=ce) for i, ce in enumerate(ces)))
    return str(path)


def test_compare_logs(tmp_path, capsys):
    a = _write(tmp_path / "a.log", [12.34, 12.30, 12.25])
    b = _write(tmp_path / "b.log", [12.341, 12.301, 12.249], t="7.9")
    c = _write(tmp_path / "c.log", [12.34, 12.30, 12.90])
    d = _write(tmp_path / "d.log", [12.34, 12.30])
    rows = compare.parse_log(a)
    assert sorted(rows) == [1, 2, 3] and rows[2]["cross-entropy-loss"] == 12.30 and rows[1]["tokens-per-second"] == 15942
    assert rows[1]["load-balance-loss"] == 1.02e-3
    assert compare.main([a, b, "--skip", "0"]) == 0
    assert "step-time" in capsys.readouterr().out
    assert compare.main([a, c]) == 1 and "step 3" in capsys.readouterr().out
    assert compare.main([a, d]) == 1


def test_profile_analyze(tmp_path, capsys):
    import gzip
    import json

    from pithtrain_b200.tools.profile import analyze

    ev = lambda name, cat, ts, dur, stream: {"ph": "X", "cat": cat, "name": name, "ts": ts, "dur": dur, "args": {"stream": stream}}
    events = [ev("pt_gemm_kernel<128>", "kernel", 0, 100, 7), ev("rmsnorm_fwd", "kernel", 100, 50, 7),
              ev("ncclDevKernel_SendRecv", "kernel", 50, 100, 13), ev("pt_gemm_kernel<128>", "kernel", 200, 100, 7),
              ev("Memcpy DtoD", "gpu_memcpy", 320, 10, 7), {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "ts": 0, "dur": 5}]
    with gzip.open(tmp_path / "trace_rank0.json.gz", "wt") as f:
        json.dump({"traceEvents": events}, f)
    r = analyze.analyze_events(analyze.load_events(tmp_path / "trace_rank0.json.gz"))
    assert r["window_us"] == 330 and r["idle_us"] == 330 - (150 + 100 + 10)
    assert r["classes"]["gemm"]["sum_us"] == 200 and r["classes"]["communication"]["launches"] == 1
    assert abs(r["comm_overlap"] - 1.0) < 1e-9 and r["streams"]["7"]["launches"] == 4
    assert r["top"][0]["name"].startswith("pt_gemm")
    assert analyze.main([str(tmp_path), "--json", str(tmp_path / "o.json")]) == 0
    assert "communication overlapped" in capsys.readouterr().out and (tmp_path / "o.json").exists()
    assert analyze.intersect([(0, 10), (20, 30)], [(5, 25)]) == 10


def test_benchmark_recipes(tmp_path):
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    from benchmarks.pretraining.recipes import MODELS, make_cfg, parse_mesh

    m = parse_mesh("h100-8n8g/pp4-dp2-cp1-ep8-seq4096-bf16-hsdp")
    assert (m["pp"], m["dp"], m["cp"], m["ep"], m["seq"], m["gpus"], m["hsdp"], m["gbs"]) == (4, 2, 1, 8, 4096, 64, True, 1024)
    assert parse_mesh("b200-1n1g/pp1-dp1-cp1-ep1-seq4096-bf16-gbs32")["gbs"] == 32
    for model, recipe in MODELS.items():
        for mesh in recipe.meshes:
            cfg = make_cfg(model, mesh, tmp_path)
            d, t = cfg.distributed, cfg.training
            pm = parse_mesh(mesh)
            assert (d.pipeline_parallel_size, d.expert_parallel_size, d.context_parallel_size) == (pm["pp"], pm["ep"], pm["cp"])
            assert t.benchmark and t.max_steps == 25 and t.sequence_length == pm["seq"] and t.dataset is None
            assert t.global_batch_size % (pm["dp"] * pm["ep"]) == 0
            assert t.global_batch_size // (pm["dp"] * pm["ep"]) >= 2 * pm["pp"]  # enough micro-batches for the V schedule
    assert "yarn" in open(tmp_path / "benchmarks" / "gpt-oss-120b" / "model.json").read()


def test_wandb_run_helpers_with_fake_api(tmp_path, capsys):
    from pithtrain_b200.tools.wandb_tracking import runs as W

    class FakeFile:
        def __init__(self, name): self.name = name
        def download(self, root, replace):
            open(f"{root}/{self.name}", "w").write("log")

    class FakeRun:
        def __init__(self, rid, name, vals):
            self.id, self.name, self.state, self.lastHistoryStep, self._v = rid, name, "finished", len(vals) - 1, vals
        def scan_history(self, keys):
            return [{"_step": i, keys[1]: v} for i, v in enumerate(self._v)]
        def file(self, name): return FakeFile(name)

    class FakeApi:
        def runs(self, project):
            return [FakeRun("aaa111", "base", [12.0, 11.5, 11.0]), FakeRun("bbb222", "feature", [12.0, 11.6, 10.9, 10.5])]

    api = FakeApi()
    assert W.main(["list", "me/proj"], api=api) == 0
    assert "2 runs" in capsys.readouterr().out
    assert W.main(["compare", "me/proj", "--metric", "train/cross-entropy-loss", "--ref", "base", "--runs", "bbb222"], api=api) == 0
    out = capsys.readouterr().out
    assert "3 common steps" in out and "max +0.1" in out and "min -0.1" in out
    assert W.main(["files", "me/proj", "--runs", "feature", "--out", str(tmp_path)], api=api) == 0
    assert (tmp_path / "feature" / "output.log").read_text() == "log"
    import pytest as _pytest
    with _pytest.raises(SystemExit):
        W.resolve(api, "me/proj", "nope")


def test_wandb_saved_views_with_fake_graphql(capsys):
    """list / create / edit / show / delete against an in-memory stand-in for the project's view store."""
    import json

    from pithtrain_b200.tools.wandb_tracking import views as V

    class Run:
        def __init__(self, id, name): self.id, self.name = id, name

    class Api:
        def runs(self, path): return [Run("r1", "base"), Run("r2", "feature"), Run("r3", "ablation")]

    store = {}

    def graphql(doc, variables):
        if "allViews" in doc:
            return {"project": {"allViews": {"edges": [{"node": dict(v)} for v in store.values()]}}}
        if "upsertView" in doc:
            inp = variables["input"]
            inserted = "id" not in inp
            vid = inp.get("id") or f"view{len(store)}"
            store[vid] = {"id": vid, "name": inp["name"], "displayName": inp["displayName"], "spec": inp["spec"]}
            assert inp["type"] == "project-view" and inp["entityName"] == "team" and inp["projectName"] == "proj"
            return {"upsertView": {"view": store[vid], "inserted": inserted}}
        if "deleteView" in doc:
            return {"deleteView": {"success": store.pop(variables["input"]["id"], None) is not None}}
        raise AssertionError(doc)

    assert V.slug_of("nw-abc123-v") == "abc123" and V.slug_of("report-7") is None and V.name_of("q") == "nw-q-v"
    assert V.main(["create", "team/proj", "--name", "base vs feature", "--runs", "base,r2"], api=Api(), graphql=graphql) == 0
    (view,) = store.values()
    slug = V.slug_of(view["name"])
    spec = json.loads(view["spec"])
    assert spec["section"]["runSets"][0]["selections"] == {"root": 1, "bounds": [], "tree": ["r3"]}
    assert V.split_runs(spec, {"r1": "base", "r2": "feature", "r3": "ablation"}) == (["base", "feature"], ["ablation"])
    # a second view copies the layout of the first and gets a link of its own
    spec["section"]["panelBankConfig"]["sections"] = [{"name": "train"}]
    view["spec"] = json.dumps(spec)
    assert V.main(["create", "team/proj", "--name", "only ablation", "--runs", "ablation", "--like", slug], api=Api(), graphql=graphql) == 0
    assert len(store) == 2
    other = [v for v in store.values() if v["displayName"] == "only ablation"][0]
    ospec = json.loads(other["spec"])
    assert ospec["section"]["panelBankConfig"]["sections"] == [{"name": "train"}]
    assert ospec["section"]["runSets"][0]["selections"]["tree"] == ["r1", "r2"]
    assert ospec["section"]["runSets"][0]["id"] != spec["section"]["runSets"][0]["id"]
    # editing keeps name (and therefore the link), changes the hide-list and optionally the title
    assert V.main(["edit", "team/proj", slug, "--runs", "r3,r1", "--name", "renamed"], api=Api(), graphql=graphql) == 0
    assert len(store) == 2 and view["id"] in store
    edited = store[view["id"]]
    assert edited["name"] == V.name_of(slug) and edited["displayName"] == "renamed"
    assert json.loads(edited["spec"])["section"]["runSets"][0]["selections"]["tree"] == ["r2"]
    capsys.readouterr()
    assert V.main(["show", "team/proj", slug], api=Api(), graphql=graphql) == 0
    out = capsys.readouterr().out
    assert "visible: ablation, base" in out and "hidden : feature" in out
    assert V.main(["list", "team/proj"], api=Api(), graphql=graphql) == 0
    assert capsys.readouterr().out.count("?nw=") == 2
    assert V.main(["delete", "team/proj", slug], api=Api(), graphql=graphql) == 0 and len(store) == 1
    with pytest.raises(SystemExit):
        V.main(["show", "team/proj", slug], api=Api(), graphql=graphql)
    with pytest.raises(SystemExit):
        V.main(["create", "team/proj", "--name", "x", "--runs", "nope"], api=Api(), graphql=graphql)


def test_benchmark_routing_generators():
    import torch

    from benchmarks.operators.utilities import make_routing, remote_rows_by_destination

    loads = {}
    for kind in ("uniform", "normal", "zipf"):
        idx = make_routing(2048, 128, 8, kind, seed=3)
        assert idx.shape == (2048, 8) and idx.dtype == torch.int32
        assert bool((idx.sort(-1).values.diff(dim=-1) > 0).all())  # k distinct experts per token
        assert torch.equal(idx, make_routing(2048, 128, 8, kind, seed=3))
        loads[kind] = torch.bincount(idx.flatten().long(), minlength=128).float()
    assert float(loads["uniform"].max() / loads["uniform"].mean()) < 1.5
    assert float(loads["normal"].max() / loads["normal"].mean()) < 1.5
    assert float(loads["zipf"].max() / loads["zipf"].mean()) > 8 and int(loads["zipf"].argmax()) == 0
    rows = remote_rows_by_destination(make_routing(1000, 16, 2, "uniform", seed=0), 16, 4, 1)
    assert int(rows[1]) == 0 and rows.shape == (4,) and int(rows.sum()) <= 2000


def test_memory_trace_follows_the_schedule(tmp_path, monkeypatch):
    import json

    from utilities import launch

    import train_worker
    from pithtrain_b200.tools import memory_trace as MT

    assert MT.ranks_from_env("") == set() and MT.ranks_from_env("0,3") == {0, 3} and MT.ranks_from_env("all") is None
    out = tmp_path / "trace.json"
    launch(2, train_worker.run_memory_trace, str(out), timeout=300.0)
    assert json.load(open(out))["rows"] > 0


def test_wandb_tracking_is_lazy_and_logs_the_metric_set(tmp_path):
    import json

    from utilities import launch

    import train_worker

    out = tmp_path / "wandb.json"
    launch(1, train_worker.run_with_fake_wandb, str(out), timeout=300.0)
    rows = json.load(open(out))
    assert len(rows) == 2 and rows[0]["train/cross-entropy-loss"] > 0


def test_tiny_cpu_benchmark_script_prints_its_json_line():
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    res = subprocess.run([sys.executable, str(root / "benchmarks" / "pretraining" / "tiny_cpu.py"), "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    row = json.loads(res.stdout.strip().splitlines()[-1])
    assert row["unit"] == "ms" and row["value"] > 0 and row["higher_is_better"] is False and 6.0 < row["final_loss"] < 7.5


def test_validation_run_recipes_build():
    from argparse import Namespace

    from pithtrain_b200.tools.validate_correctness.validate import RECIPES, make_cfg

    for model in RECIPES:
        a = Namespace(model=model, pipeline_parallel_size=2, expert_parallel_size=4, context_parallel_size=1, synthetic=True,
                      max_steps=25, global_batch_size=1024, sequence_length=2048, fp8=False, num_hidden_layers=0)
        cfg = make_cfg(a)
        t = cfg.training
        assert t.dataset is None and t.lr == 1e-6 and t.max_steps == 25 and t.model.name == "config.json"
        assert (ROOT_DIR / t.model).exists(), t.model
        assert t.moe_load_balance_type in ("sequence", "global-batch", "micro-batch")


def test_profile_analyzer_classifies_the_framework_kernels():
    from pithtrain_b200.tools.profile.analyze import classify

    cases = {
        "pt::ep_push_kernel(pt::EpChan, int, unsigned int, ...)": "communication",
        "pt::ep_compact_kernel(pt::EpChan, int, int const*, ...)": "communication",
        "pt::fsdp::reduce_scatter_kernel(pt::fsdp::Chan, ...)": "communication",
        "pt::fsdp::wait_kernel(pt::fsdp::Chan, int, unsigned int, int*)": "communication",
        "ncclDevKernel_SendRecv(ncclDevKernelArgsStorage<4096ul>)": "communication",
        "void pt::gemm_bf16_kernel<256, true, true, false, true>(CUtensorMap_st, ...)": "gemm",
        "pt::gemm2cta_kernel(CUtensorMap_st, CUtensorMap_st, CUtensorMap_st, pt::Gemm2Args)": "gemm",
        "nvjet_tst_256x256_64x4_2x1_2cta_v_bx_NNT": "gemm",
        "pt::attn_fwd_kernel(CUtensorMap_st, CUtensorMap_st, CUtensorMap_st, pt::AttnArgs)": "attention",
        "cudnn_generated_fort_native_sdpa_sm100_flash_bprop_f16_knob_31_128x128x128": "attention",
        "pt::muon_momentum_kernel(...)": "optimizer",
        "pt::rmsnorm_fwd_kernel<8>(...)": "other",
    }
    for name, want in cases.items():
        assert classify(name, "kernel") == want, (name, classify(name, "kernel"))
    assert classify("Memcpy DtoD (Device -> Device)", "gpu_memcpy") == "memcpy"


def test_profile_analyzer_reads_nsight_systems_sqlite_exports(tmp_path, capsys):
    """A synthetic export with the tables the reader uses: kernels on a compute and a communication stream, launch
    records, NVTX stage ranges and the ``rank=`` window opened by ``nsys_start``."""
    import sqlite3

    from pithtrain_b200.tools.profile import analyze as A

    db_path = tmp_path / "rank0.sqlite"
    db = sqlite3.connect(db_path)
    db.executescript("""
        CREATE TABLE StringIds (id INTEGER PRIMARY KEY, value TEXT);
        CREATE TABLE CUPTI_ACTIVITY_KIND_KERNEL (start INT, end INT, deviceId INT, streamId INT, correlationId INT, demangledName INT, shortName INT);
        CREATE TABLE CUPTI_ACTIVITY_KIND_MEMCPY (start INT, end INT, deviceId INT, streamId INT, correlationId INT, bytes INT, copyKind INT);
        CREATE TABLE CUPTI_ACTIVITY_KIND_RUNTIME (start INT, end INT, globalTid INT, correlationId INT, nameId INT);
        CREATE TABLE NVTX_EVENTS (start INT, end INT, eventType INT, text TEXT, globalTid INT, textId INT);
    """)
    names = {1: "void pt::gemm_bf16_kernel<256, false, false, false, false>(CUtensorMap_st)", 2: "pt::ep_push_kernel(pt::EpChan)",
             3: "pt::rmsnorm_fwd_kernel<8>()", 4: "layer03.stage2_f"}
    db.executemany("INSERT INTO StringIds VALUES (?, ?)", names.items())
    us = 1000
    # (start, end, stream, corr, name id): a GEMM on stream 7 overlapping a push on stream 9; one kernel before the window
    kernels = [(100 * us, 200 * us, 7, 11, 1), (120 * us, 180 * us, 9, 12, 2), (210 * us, 220 * us, 7, 13, 3), (10 * us, 20 * us, 7, 14, 3)]
    db.executemany("INSERT INTO CUPTI_ACTIVITY_KIND_KERNEL VALUES (?, ?, 0, ?, ?, ?, ?)", [(s, e, st, c, n, n) for s, e, st, c, n in kernels])
    db.execute("INSERT INTO CUPTI_ACTIVITY_KIND_MEMCPY VALUES (?, ?, 0, 7, 15, 4096, 8)", (230 * us, 232 * us))
    launches = [(95 * us, 11), (115 * us, 12), (205 * us, 13), (5 * us, 14), (228 * us, 15)]
    db.executemany("INSERT INTO CUPTI_ACTIVITY_KIND_RUNTIME VALUES (?, ?, 42, ?, 0)", [(s, s + 2 * us, c) for s, c in launches])
    nvtx = [(50 * us, 300 * us, "rank=0; pp=0/1 dp=0/1 cp=0/1 ep=0/2; mbs=1 seq=4096", None),
            (90 * us, 110 * us, "layer03.stage1_f", None), (112 * us, 118 * us, None, 4), (200 * us, 209 * us, "layer03.stage3_f", None)]
    db.executemany("INSERT INTO NVTX_EVENTS VALUES (?, ?, 59, ?, 42, ?)", nvtx)
    db.commit()
    db.close()

    events = A.load_events_sqlite(db_path)
    assert len(events) == 4  # the kernel before the rank= window is dropped
    r = A.analyze_events(events)
    assert abs(r["window_us"] - 132.0) < 1e-6
    assert r["classes"]["gemm"]["sum_us"] == 100.0 and r["classes"]["communication"]["sum_us"] == 60.0
    assert r["comm_overlap"] == 1.0  # the push ran entirely under the GEMM
    assert set(r["stages"]) == {"stage1_f", "stage2_f", "stage3_f"}
    assert r["stages"]["stage2_f"]["comm_us"] == 60.0 and r["stages"]["stage2_f"]["comm_overlap"] == 1.0
    assert r["stages"]["stage1_f"]["sum_us"] == 100.0 and r["stages"]["stage3_f"]["launches"] == 1
    assert A.main([str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "stage2_f" in out and "communication overlapped with compute: 100.0%" in out


def test_profile_analyzer_attributes_kernels_to_stage_annotations(tmp_path):
    """A trace captured with ``--with-cpu``: stage ranges are ``user_annotation`` events on the launching thread and
    kernels are tied to their launch through the correlation id."""
    import json

    from pithtrain_b200.tools.profile import analyze as A

    ev = [
        {"ph": "X", "cat": "user_annotation", "name": "layer00.stage1_f", "pid": 1, "tid": 5, "ts": 100.0, "dur": 50.0},
        {"ph": "X", "cat": "user_annotation", "name": "layer00.stage3_w", "pid": 1, "tid": 5, "ts": 160.0, "dur": 20.0},
        {"ph": "X", "cat": "user_annotation", "name": "profiled_step", "pid": 1, "tid": 5, "ts": 90.0, "dur": 500.0},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "pid": 1, "tid": 5, "ts": 110.0, "dur": 3.0, "args": {"correlation": 71}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "pid": 1, "tid": 5, "ts": 165.0, "dur": 3.0, "args": {"correlation": 72}},
        {"ph": "X", "cat": "cuda_runtime", "name": "cudaLaunchKernel", "pid": 1, "tid": 5, "ts": 300.0, "dur": 3.0, "args": {"correlation": 73}},
        {"ph": "X", "cat": "kernel", "name": "pt::rmsnorm_fwd_kernel<8>()", "pid": 0, "tid": 7, "ts": 400.0, "dur": 10.0, "args": {"stream": 7, "correlation": 71}},
        {"ph": "X", "cat": "kernel", "name": "void pt::gemm_bf16_kernel<256, true, true, false, true>()", "pid": 0, "tid": 7, "ts": 420.0, "dur": 30.0,
         "args": {"stream": 7, "correlation": 72}},
        {"ph": "X", "cat": "kernel", "name": "pt::muon_momentum_kernel()", "pid": 0, "tid": 7, "ts": 460.0, "dur": 5.0, "args": {"stream": 7, "correlation": 73}},
    ]
    path = tmp_path / "trace_rank0.json"
    path.write_text(json.dumps({"traceEvents": ev}))
    r = A.analyze_events(A.load_events(path))
    assert r["stages"]["stage1_f"]["sum_us"] == 10.0 and r["stages"]["stage3_w"]["sum_us"] == 30.0
    assert set(r["stages"]) == {"stage1_f", "stage3_w"}  # the optimizer kernel was launched outside any stage range
    assert any("stage3_w" in line for line in A.render("rank0", r))


def test_stage_ranges_become_profiler_annotations_when_recording():
    import torch
    from torch.profiler import ProfilerActivity, profile

    from pithtrain_b200.dualpipe import execution

    assert execution.RECORD_RANGES is False
    execution.RECORD_RANGES = True
    try:
        with profile(activities=[ProfilerActivity.CPU]) as prof:
            with execution.nvtx_range("layer05.stage3_f"):
                torch.ones(4) + 1
    finally:
        execution.RECORD_RANGES = False
    assert any(e.name == "layer05.stage3_f" for e in prof.events())
    with execution.nvtx_range("layer05.stage3_f"):  # default path: no CUDA here, plain pass-through
        pass


def test_ncu_table_from_a_raw_page_export(tmp_path, capsys):
    from pithtrain_b200.tools.profile import ncu_table as T

    header = ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum",
              "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
              "sm__throughput.avg.pct_of_peak_sustained_elapsed", "launch__registers_per_thread", "launch__shared_mem_per_block_dynamic",
              "launch__grid_size", "launch__block_size", "lts__t_sector_hit_rate.pct",
              "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
              "smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio",
              "smsp__average_warps_issue_stalled_selected_per_issue_active.ratio"]
    units = ["", "", "us", "Mbyte", "Mbyte", "%", "%", "%", "register/thread", "Kbyte/block", "", "", "%", "", "", ""]
    row = ["0", "pt::rmsnorm_fwd_kernel<8>(...)", "10.00", "32.0", "32.0", "71.5", "0", "40.1", "32", "0", "4,096", "256", "12.5", "6.3", "1.2", "1.0"]
    path = tmp_path / "raw_rmsnorm.csv"
    path.write_text("==PROF== some banner line\n" + "\n".join(",".join(f'"{c}"' for c in r) for r in (header, units, row)) + "\n")
    (d,) = T.parse_raw_csv(path.read_text())
    assert d["time"] == ("10.00", "us") and d["kernel"][0].startswith("pt::rmsnorm") and d["stalls"][0] == "long_scoreboard 6.3, barrier 1.2"
    assert T.main(["--csv", str(path), "--bytes", str(64e6)]) == 0
    out = capsys.readouterr().out
    assert "| raw_rmsnorm | pt::rmsnorm_fwd_kernel<8>(...) | 10.00 us | 32.0 Mbyte / 32.0 Mbyte | 71.5 %" in out
    assert "HBM" in out and "4,096 x 256" in out
    # 64 MB in 10 us = 6400 GB/s
    frac = float(out.strip().splitlines()[-1].split("|")[-2].split()[0])
    assert 0.9 < frac < 1.05
