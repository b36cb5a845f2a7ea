"""Multi-GPU equivalence tests: fused communication kernels vs NCCL baselines vs one GPU.
Each test launches torchrun with one process per GPU; skipped with fewer than 2 GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(what, tmp_path, nproc=2, port=29611):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    out = tmp_path / f"{what}.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker.py"), what, str(out)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads(out.read_text())


def test_fused_sharded_adamw_two_gpus(tmp_path):
    res = _run("fsdp", tmp_path)
    for k, v in res.items():
        if k.endswith("fused_vs_nccl"):
            assert v < 2e-3, res
        if k.endswith("fused_vs_single"):
            assert v < 5e-3, res
        if k.endswith("gnorm_rel"):
            assert v < 1e-2, res
        if k.startswith("ckpt_"):
            assert v < 5e-3, res
    assert res["rank_checksum_spread"] == 0.0, res


def test_fused_sharded_adamw_multimem_two_gpus(tmp_path):
    """The NVLS variant (multimem.ld_reduce / multimem.st through the switch) against the NCCL baseline and one GPU."""
    res = _run("fsdp_multimem", tmp_path, port=29621)
    for k, v in res.items():
        if k.endswith("fused_vs_nccl"):
            assert v < 2e-3, res
        if k.endswith("fused_vs_single"):
            assert v < 5e-3, res
    assert res["rank_checksum_spread"] == 0.0, res


def test_checkpoint_manager_saves_trained_sharded_state_two_gpus(tmp_path):
    res = _run("ckpt_manager", tmp_path, port=29622)
    assert res["ckpt_params_vs_single"] < 5e-3 and res["ckpt_mu_vs_single"] < 5e-3, res
    assert res["moved_from_init"] > 1e-4, res


def test_pipeline_1f1b_gpt2_over_nccl_two_gpus(tmp_path):
    """PP = 2 over NCCL p2p == one GPU: loss and the gradients of both stages' blocks."""
    res = _run("pp", tmp_path, port=29623)
    assert res["stage_grad_rel"] < 3e-2 and res["loss_abs_err"] < 2e-2, res


def test_tp_fused_gemms_two_gpus(tmp_path):
    res = _run("tp", tmp_path, port=29612)
    assert res and all(v < (3e-2 if k.startswith("tp_pair_d") else 1e-2) for k, v in res.items()), res


def test_tp_fused_gemms_four_gpus(tmp_path):
    res = _run("tp", tmp_path, nproc=4, port=29622)
    assert res and all(v < (3e-2 if k.startswith("tp_pair_d") else 1e-2) for k, v in res.items()), res
    res = _run("fsdp_ag", tmp_path, nproc=4, port=29623)
    assert all(v < 1e-2 for v in res.values()), res


def test_gpt2_sequence_parallel_on_fused_gemms_two_gpus(tmp_path):
    res = _run("sp", tmp_path, port=29625)
    assert res["sp_loss_abs"] < 2e-2 and res["sp_sharded_grad_rel"] < 6e-2 and res["sp_replicated_grad_rel"] < 6e-2, res


def test_context_parallel_attention_two_gpus(tmp_path):
    res = _run("cp", tmp_path, port=29624)
    assert res and all(v < 3e-2 for v in res.values()), res


def test_fsdp_all_gather_fused_into_gemm_two_gpus(tmp_path):
    res = _run("fsdp_ag", tmp_path, port=29614)
    assert all(v < 1e-2 for v in res.values()), res


def test_fused_ep_moe_two_gpus(tmp_path):
    res = _run("ep", tmp_path, port=29613)
    for k, v in res.items():
        if k.endswith("_vs_dense"):
            assert v < 2e-2, res


def test_fused_ep_moe_backward_two_gpus(tmp_path):
    res = _run("ep_bwd", tmp_path, port=29615)
    for k, v in res.items():
        assert v < 3e-2, res


def test_tensor_parallel_attention_layers_two_gpus(tmp_path):
    res = _run("tp_attention", tmp_path, port=29619)
    assert res["mla_tp"] < 2e-2 and res["gqa_tp"] < 2e-2, res


def test_vocab_parallel_cross_entropy_two_gpus(tmp_path):
    res = _run("vocab_ce", tmp_path, port=29618)
    for k, v in res.items():
        assert v < (2e-2 if k.startswith("dw") else 3e-3), res


def test_fused_ep_moe_fp8_two_gpus(tmp_path):
    res = _run("ep_fp8", tmp_path, port=29617)
    for k, v in res.items():
        if k.endswith("_vs_quantised_ref"):
            assert v < 2e-2, res
        if k.endswith("_vs_bf16_math"):
            assert v < 1e-1, res


@pytest.mark.parametrize("nproc", [4, 8])
def test_fused_ep_moe_forward_backward_fp8_more_gpus(tmp_path, nproc):
    """The expert-parallel kernels with 4 and 8 ranks (16 experts: 4 and 2 per rank): forward against the dense
    evaluation, backward against autograd of it, the FP8 forward against its quantised restatement."""
    res = _run("ep", tmp_path, nproc=nproc, port=29631)
    assert all(v < 2e-2 for k, v in res.items() if k.endswith("_vs_dense")), res
    res = _run("ep_bwd", tmp_path, nproc=nproc, port=29632)
    assert all(v < 3e-2 for v in res.values()), res
    res = _run("ep_fp8", tmp_path, nproc=nproc, port=29633)
    assert all(v < 2e-2 for k, v in res.items() if k.endswith("_vs_quantised_ref")), res


def test_qwen35_expert_parallel_training_matches_single_process(tmp_path):
    res = _run("moe_train", tmp_path, port=29616)
    assert res["ep_loss"][0] > 5.5                      # ln(512) = 6.24 at random init
    assert res["ref_loss"][-1] < res["ref_loss"][0], res
    assert res["ep_loss"][-1] < res["ep_loss"][0], res
    for a, b in zip(res["ep_loss"], res["ref_loss"]):
        assert abs(a - b) < 0.05 * b, res
    for a, b in zip(res["gnorm_ep"], res["gnorm_ref"]):
        assert abs(a - b) < 0.1 * b + 1e-3, res


def test_bounded_wait_reports_timeout(cuda_device):
    """A flag that nothing sets: the kernel gives up after its budget, records the status
    and returns; the context stays usable."""
    from jax_gpt_b200 import _ext
    flag = torch.zeros(1, device=cuda_device, dtype=torch.int32)
    _ext.ops().wait_flag(flag, 1, 0.2)
    with pytest.raises(_ext.KernelStatusError):
        _ext.check_status(cuda_device)
    # the device still works and the status word was reset
    assert float((torch.ones(4, device=cuda_device) * 2).sum()) == 8.0
    _ext.check_status(cuda_device)
    flag.fill_(3)
    _ext.ops().wait_flag(flag, 1, 0.2)
    _ext.check_status(cuda_device)
