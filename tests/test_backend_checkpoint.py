"""State compatibility through backend="gpubridge": object collectives in every direction and a
torch.distributed.checkpoint save / load of an FSDP2-sharded model (planning uses
gather_object / scatter_object_list over the backend); the state dict keys are the plain
module's (no wrapper modules are added)."""
import torch

from _harness import TWO_BY_TWO, run_ranks


def _objects_and_checkpoint(rank, world, folder):
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_model_state_dict, set_model_state_dict
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    objs = [None] * world
    dist.all_gather_object(objs, {"rank": rank, "name": f"r{rank}"})
    assert [o["rank"] for o in objs] == list(range(world))
    got = [None]
    dist.scatter_object_list(got, [f"for-{r}" for r in range(world)] if rank == 1 else None, src=1)
    assert got[0] == f"for-{rank}"
    box = [{"payload": list(range(5))}] if rank == 2 else [None]
    dist.broadcast_object_list(box, src=2)
    assert box[0] == {"payload": [0, 1, 2, 3, 4]}
    gathered = [None] * world if rank == 3 else None
    dist.gather_object(("x", rank), gathered, dst=3)
    if rank == 3:
        assert gathered == [("x", r) for r in range(world)]

    def make(seed):
        torch.manual_seed(seed)
        return torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))

    mesh = init_device_mesh("cpu", (world,))
    model = make(0)
    plain_keys = list(model.state_dict())
    for layer in model:
        if isinstance(layer, torch.nn.Linear):
            fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    assert list(model.state_dict()) == plain_keys
    full_before = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    dcp.save({"model": get_model_state_dict(model)}, checkpoint_id=folder)
    other = make(1)                                   # different weights, same sharding
    for layer in other:
        if isinstance(layer, torch.nn.Linear):
            fully_shard(layer, mesh=mesh)
    fully_shard(other, mesh=mesh)
    state = {"model": get_model_state_dict(other)}
    dcp.load(state, checkpoint_id=folder)
    set_model_state_dict(other, state["model"])
    for k, v in other.state_dict().items():
        assert torch.equal(v.full_tensor(), full_before[k]), k
    dist.barrier()
    return True


def test_object_collectives_and_distributed_checkpoint(tmp_path):
    folder = str(tmp_path / "ckpt")
    run_ranks(TWO_BY_TWO, _objects_and_checkpoint, tmp_path, folder, mode="backend", timeout=240)
