"""CPU tests of the level-3 (multi-GPU) launch surface: ``DistributedConfig`` constraints
(python/pypto/ir/distributed_compiled_program.py:87-117 of the reference), ``ir.compile(distributed_config=...)``
-> ``DistributedCompiledProgram``, argument checks of the one-shot call, and -- when the reference tree is
present -- its own expert-parallel test module imported and compiled unchanged."""

import importlib.util
import os

import pytest
import torch

import ep_program
from pypto_b200 import BackendUnavailable, ir
from pypto_b200.ir import DistributedCompiledProgram, DistributedConfig
from pypto_b200.runtime import DeviceTensor


def test_distributed_config_constraints():
    assert DistributedConfig().device_ids == [0]
    for bad in ([], [-1], [0, 0]):
        with pytest.raises(ValueError):
            DistributedConfig(device_ids=bad)
    with pytest.raises(ValueError):
        DistributedConfig(num_sub_workers=-1)
    with pytest.raises(ValueError):
        DistributedConfig(aicpu_thread_num=1)
    assert DistributedConfig(device_ids=[3, 1], aicpu_thread_num=2).device_ids == [3, 1]


def test_compile_resolves_the_host_orchestrator():
    prog = ep_program.build(2, 16, 3, 32, 4, 40)
    assert prog.host_entry.name == "host_orch" and prog.entry is prog.host_entry
    c = ir.compile(prog, platform="b200", distributed_config=DistributedConfig(device_ids=[0, 1]))
    assert isinstance(c, DistributedCompiledProgram) and c.world_size == 2 and c.platform == "b200"
    with pytest.raises(TypeError):
        ir.compile(prog, platform="b200", distributed_config={"device_ids": [0, 1]})
    with pytest.raises(BackendUnavailable):
        ir.compile(prog, platform="a2a3", distributed_config=DistributedConfig(device_ids=[0, 1]))


def test_one_shot_call_argument_checks():
    c = ir.compile(ep_program.build(2, 16, 3, 32, 4, 40), platform="b200",
                   distributed_config=DistributedConfig(device_ids=[0, 1]))
    with pytest.raises(TypeError, match="10"):
        c(torch.zeros(1))
    args = ep_program.host_tensors(torch.zeros(2, 16, 32, dtype=torch.bfloat16), torch.zeros(2, 16, 3),
                                   torch.zeros(2, 16, 3, dtype=torch.int32), 4, 40)
    with pytest.raises(TypeError, match="DeviceTensor"):
        c(DeviceTensor(16, (2, 16, 3), torch.int32), *args[1:])
    with pytest.raises(TypeError, match="host torch.Tensor"):
        c(*args[:3], "idx", *args[4:])
    if not torch.cuda.is_available():
        with pytest.raises(BackendUnavailable):       # no GPUs here: the worker refuses, nothing falls back to the CPU
            c(*args)


def test_rank_side_validation_of_stacked_shapes():
    from pypto_b200.runtime import distributed_programs
    op = distributed_programs.lookup(ep_program.build(2, 16, 3, 32, 4, 40).host_entry)
    names = distributed_programs.EpDispatchCombineOp.names
    args = ep_program.host_tensors(torch.zeros(2, 16, 32, dtype=torch.bfloat16), torch.zeros(2, 16, 3),
                                   torch.zeros(2, 16, 3, dtype=torch.int32), 4, 40)
    op.validate(2, dict(zip(names, args)))
    bad = list(args)
    bad[0] = torch.full((2, 16, 3), 8, dtype=torch.int32)           # expert id 8 with 2 x 4 experts
    with pytest.raises(ValueError, match="expert ids"):
        op.validate(2, dict(zip(names, bad)))
    with pytest.raises(ValueError, match="leading dimension"):
        op.validate(4, dict(zip(names, args)))
    bad = list(args)
    bad[8] = torch.zeros(2, 4 * 40, 16, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="recv_ys"):
        op.validate(2, dict(zip(names, bad)))


def test_unknown_host_entry_has_no_kernel():
    import pypto_b200.language as pl

    @pl.program
    class Other:
        @pl.function(level=pl.Level.HOST, role=pl.Role.Orchestrator)
        def host_orch(self, a: pl.Tensor[[2, 4], pl.FP32], b: pl.Out[pl.Tensor[[2, 4], pl.FP32]]):
            ...

    with pytest.raises(NotImplementedError, match="no multi-GPU kernel"):
        ir.compile(Other, platform="b200", distributed_config=DistributedConfig(device_ids=[0, 1]))


def test_reference_ep_test_module_imports_and_compiles_unchanged():
    import ref_extract
    path = os.path.join(ref_extract.REFERENCE_ROOT, "tests", "st", "distributed", "test_l3_ep_dispatch_combine.py")
    if not os.path.exists(path):
        pytest.skip("reference tree not mounted")
    from pypto_b200 import compat
    compat.install()
    spec = importlib.util.spec_from_file_location("reference_ep_dispatch_combine", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for n_ranks in (2, 4):
        prog = mod._build_ep_dispatch_combine_program(n_ranks)
        c = mod.ir.compile(prog, platform="b200",
                           distributed_config=mod.DistributedConfig(device_ids=list(range(n_ranks)), num_sub_workers=0))
        assert isinstance(c, DistributedCompiledProgram) and c.world_size == n_ranks
        assert [p.name for p in c.params][:4] == ["indices", "x_norms", "w_padded", "idx_padded"]
