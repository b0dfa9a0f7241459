"""Host-side checks of the profiling tools (no GPU): the GPU spec table and
profile loader, the YAML generator, and the ncu command-line helper — the
behaviours of the reference's scripts/roofline_profile.py, scripts/ncu_profile.py
and benchmarks/hardware/gpu_specs.py that a user relies on."""

import importlib.util
import sys
from pathlib import Path

import pytest
import yaml

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from benchmarks.hardware import gpu_specs  # noqa: E402


def _load(name):
    spec = importlib.util.spec_from_file_location(name, ROOT / "benchmarks" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_detect_profile_matches_name_variants():
    assert gpu_specs.detect_profile("NVIDIA B200") == "b200"
    assert gpu_specs.detect_profile("NVIDIA B200 180GB HBM3e") == "b200"
    assert gpu_specs.detect_profile("NVIDIA B2") == "b200"  # reverse prefix, as the reference matches
    assert gpu_specs.detect_profile("Some Other GPU") is None
    assert gpu_specs.get_specs("b200")["hbm_bw_gb"] == 8000.0
    assert gpu_specs.get_specs("nope") is None


def test_committed_b200_profile_loads_with_effective_values():
    p = gpu_specs.load_profile("b200")
    assert p["gpu"] == "NVIDIA B200" and p["sm_count"] == 148
    assert p["hbm"]["theoretical"] == 8000e9
    assert p["hbm"]["effective"] == pytest.approx(p["hbm"]["theoretical"] * p["hbm"]["calibration"])
    for dtype in ("bf16", "fp16", "tf32", "fp8"):
        node = p["tensor_core"][dtype]
        assert node["effective"] == pytest.approx(node["theoretical"] * node["calibration"])
    assert gpu_specs.load_profile("no_such_gpu") is None


def test_generate_yaml_round_trips_and_marks_placeholders(tmp_path):
    rp = _load("roofline_profile")
    specs = gpu_specs.get_specs("b200")
    text = rp.generate_yaml("NVIDIA B200", "10.0", 148, 126 << 20, 228 << 10,
                            {"theoretical_gbs": 8000.0, "calibration": 0.80612},
                            {"bf16": {"calibration": 0.7555}}, specs)
    data = yaml.safe_load(text)
    assert data["hbm"] == {"theoretical": "8000e9", "calibration": 0.806} or float(data["hbm"]["theoretical"]) == 8000e9
    assert data["tensor_core"]["bf16"]["calibration"] == 0.76
    assert data["tensor_core"]["fp8"]["calibration"] == 0.76  # placeholder = first measured calibration
    assert "placeholder" in text and text.count("placeholder") == 3
    (tmp_path / "b200.yaml").write_text(text)
    loaded = gpu_specs.load_profile("b200", assets_dir=tmp_path)
    assert loaded["hbm"]["effective"] == pytest.approx(8000e9 * 0.806)
    assert loaded["tensor_core"]["tf32"]["theoretical"] == 1125e12
    assert rp._sci(2250.5, 12) == "2250.5e12" and rp._sci(8000.0, 9) == "8000e9"


def test_ncu_cli_helpers():
    nc = _load("ncu_profile")
    assert nc.op_name_to_class("qwen3_dense_decode") == "Qwen3DenseDecodeOp"
    assert nc.op_name_to_class("gemv") == "GemvOp"
    assert nc.parse_params("N=4096,K=4096") == ([], {"N": 4096, "K": 4096})
    assert nc.parse_params("32, 4096, 1e-6") == ([32, 4096, 1e-6], {})
    assert nc.parse_params("") == ([], {})
    script = nc.generate_profile_script("gemv", "cuda", [], {"N": 4096, "K": 1024})
    assert "GemvOp(N=4096, K=1024, backend='cuda')" in script and "op(*data)" in script
    compile(script, "<profile script>", "exec")
    ref_script = nc.generate_profile_script("rmsnorm", "ref", [8, 512], {})
    assert "RmsNormOp(8, 512)" in ref_script and "op._ref_forward(*data)" in ref_script
    cmd = nc.ncu_command("ncu", Path("out/x"), Path("run.py"), 2, "gemv")
    assert cmd[:5] == ["ncu", "--set", "full", "--clock-control", "none"]  # never lock the clocks of a shared GPU
    assert cmd[cmd.index("-c") + 1] == "2" and "regex:gemv" in cmd


def test_every_op_class_resolves_from_its_snake_case_name():
    import ezops_b200 as ez

    nc = _load("ncu_profile")
    for op in ez.list_ops():
        assert hasattr(ez, nc.op_name_to_class(op)), op


def test_per_operator_benchmark_scripts_keep_the_reference_command_line():
    """``python benchmarks/bench_<op>.py -h`` lists the backends and exits; an unknown backend is refused with the
    list (ezops benchmarks/bench_gemv.py:177-212).  Neither touches a GPU."""
    import subprocess
    import sys
    from pathlib import Path

    bench_dir = Path(__file__).resolve().parent.parent / "benchmarks"
    for script, expect in (("bench_gemv.py", "cuda"), ("bench_rmsnorm.py", "cuda"), ("bench_fused_qk_norm_rope.py", "cuda"),
                           ("bench_attn_decode.py", "cuda"), ("bench_fused_o_proj_ffn.py", "cuda"),
                           ("bench_qwen3_dense_decode.py", "cuda"), ("bench_pdl_gemm.py", "cuda, cuda_pdl")):
        res = subprocess.run([sys.executable, str(bench_dir / script), "-h"], capture_output=True, text=True, timeout=120, cwd=str(bench_dir))
        assert res.returncode == 0, res.stderr[-500:]
        assert res.stdout.strip() == f"Available backends: {expect}", res.stdout
    res = subprocess.run([sys.executable, str(bench_dir / "bench_gemv.py"), "-k", "triton"], capture_output=True, text=True, timeout=120,
                         cwd=str(bench_dir))
    assert "Unknown backends: triton" in res.stdout and "Available: cuda" in res.stdout


def test_gemv_timeline_script_parses_its_command_line_without_a_gpu():
    import subprocess
    import sys
    from pathlib import Path

    script = Path(__file__).resolve().parent.parent / "benchmarks" / "gemv_isolated_timeline.py"
    res = subprocess.run([sys.executable, str(script), "--help"], capture_output=True, text=True, timeout=180)
    assert res.returncode == 0, res.stderr[-500:]
    assert "--rows" in res.stdout and "--launches" in res.stdout
