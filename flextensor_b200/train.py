"""Offline training of the walkers' Q-networks and of the performance model from dumped search
data (counterpart of flextensor/train.py:13-58,123-...: the reference trains from the JSON-lines
files `WalkerGroup.dump_data` writes, then `schedule(..., op_perf_model_path=...)` searches against
the trained performance model instead of measuring).

    python -m flextensor_b200.train --task "gemm_batch_gemm_(4, 256, 512, 384)_cuda(0)" --op 0 --what walker
    python -m flextensor_b200.train --task ... --op 0 --what perf
"""
import argparse

from .model import WalkerGroup
from .scheduler import flatten_graph
from .space import generate_space_intra_op
from .task import TASK_TABLE


def group_for(task_key, op_pos):
    """The walker group a search of ``task_key`` builds for op ``op_pos`` (same names, hence the
    same checkpoint and data file names)."""
    task = TASK_TABLE[task_key]
    ops, _ = task.func(*task.args)
    op_lst, down_graph = flatten_graph(ops)
    space = generate_space_intra_op(op_lst[op_pos], down_graph, target=task.target)
    return WalkerGroup(task.category + "_op" + str(op_pos), space)


def train_walkers(task_key, op_pos, verbose=True):
    """Load dumped (state, action, next state, reward) tuples, train every sub-space's Q-network,
    save the checkpoints (the target network is synced on save)."""
    group = group_for(task_key, op_pos)
    group.load_walker_model()
    group.load_walker_data()
    group.train_walkers(save=True, verbose=verbose)
    return group


def train_performance(task_key, op_pos, verbose=True):
    """Load dumped (points, costs) batches, train the ranking performance model, save it; returns
    the group and its mean ranking loss on the data."""
    group = group_for(task_key, op_pos)
    group.load_or_create_model()
    group.prepare_performance_data()
    group.train_on_perf(save=True, verbose=verbose)
    return group, group.test_accuracy()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--task", required=True, help="task key")
    parser.add_argument("--op", type=int, default=0, help="position of the op in the flattened graph")
    parser.add_argument("--what", choices=["walker", "perf"], default="perf")
    args = parser.parse_args()
    if args.what == "walker":
        train_walkers(args.task, args.op)
    else:
        _, loss = train_performance(args.task, args.op)
        print("ranking loss %.6f" % loss)


if __name__ == "__main__":
    main()
