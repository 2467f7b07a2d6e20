"""Host-side checkpoint faults: a missing tensor-parallel shard, a tensor-parallel degree that
does not match the checkpoint's, and a truncated file each end in a clear error, never in a
half-loaded model."""
import os
import shutil

import pytest
import torch

import mp_workers as W


@pytest.fixture()
def saved(tmp_path):
    """One checkpoint of the tiny model written through checkpoint_utils (TP = 1)."""
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.parallel.fsdp import ShardedDataParallel
    from easy_to_hard_b200.utils import checkpoint_utils as cu
    from easy_to_hard_b200.utils.memory_efficient_adam import MemoryEfficientAdamW
    tpm.initialize_model_parallel(1)
    model = W.tiny_model()
    model.requires_grad_(True)
    names = [n for n, p in model.named_parameters() if p.requires_grad]
    sdp = ShardedDataParallel(model, process_group=None)
    opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=1e-3,
                               optim_dtype=torch.float32, optim_device=torch.device("cpu"))
    path = cu.get_checkpoint_path(str(tmp_path), 0, 2, 0, "")
    cu.save_checkpoint(path, sdp, opt, None, 0, 2, 0, False, None, True, names, "", None,
                       torch.float32)
    return tmp_path, path, sdp, opt


def test_resume_with_another_tensor_parallel_degree_is_refused(saved):
    from easy_to_hard_b200.utils import checkpoint_utils as cu
    d, path, sdp, opt = saved
    shutil.copy(path, path.replace("_rank_0", "_rank_1"))      # looks like a TP = 2 checkpoint
    with pytest.raises(ValueError, match="model parallel setting"):
        cu.load_checkpoint(path, sdp, opt, None, use_fsdp=True)


def test_missing_shard_is_reported_by_name(saved):
    from easy_to_hard_b200.utils import checkpoint_utils as cu
    d, path, sdp, opt = saved
    found, _, step = cu.get_latest_checkpoint_path(str(d))
    assert found == path and step == 2
    os.remove(path)
    # the pointer file still names the checkpoint; with no shard left the degree check fires
    with pytest.raises((cu.CheckpointError, ValueError)):
        cu.load_checkpoint(found, sdp, opt, None, use_fsdp=True)
    with pytest.raises(cu.CheckpointError, match="does not exist"):
        cu.read_checkpoint_file(found)
    with pytest.raises(cu.CheckpointError, match="does not exist"):
        cu.load_inference_checkpoint(found, sdp.module if hasattr(sdp, "module") else sdp)


def test_truncated_file_is_a_clean_error_and_leaves_the_model_untouched(saved):
    from easy_to_hard_b200.utils import checkpoint_utils as cu
    d, path, sdp, opt = saved
    before = {k: v.clone() for k, v in sdp.full_state_dict(rank0_only=False).items()}
    size = os.path.getsize(path)
    with open(path, "r+b") as fh:
        fh.truncate(size // 2)
    with pytest.raises(cu.CheckpointError, match="truncated or corrupt"):
        cu.load_checkpoint(path, sdp, opt, None, use_fsdp=True)
    after = sdp.full_state_dict(rank0_only=False)
    assert all(torch.equal(before[k], after[k]) for k in before)


def test_save_never_leaves_a_partial_file(saved):
    """Shards are written under a temporary name and renamed: the directory holds the finished
    file and the pointer, nothing else."""
    d, path, _, _ = saved
    names = sorted(os.listdir(d))
    assert names == ["epoch_0_step_2_rank_0.pt", "last_checkpoint"], names
