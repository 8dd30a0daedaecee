"""Q-learning walkers and the performance model that steer the search (PyTorch, CPU).

Behaviour follows the reference's ``flextensor/model.py``:
  Judger            MLP, `depth` linear layers of `width` units            (model.py:20-36)
  Walker            one DQN per sub-space: online + target net, replay memory,
                    epsilon-greedy `walk`, exhaustive `full_walk`, `train`  (model.py:39-169)
  MemEntity         heap item ordered by measured milliseconds             (model.py:172-178)
  rank_loss         pairwise logistic ranking loss                         (model.py:181-189)
  PerformanceModel  6-layer MLP predicting cost from the flattened point   (model.py:192-232)
  WalkerGroup       the walkers of a space + heap memory of visited points (model.py:235-509)
Constants kept: epsilon floor 0.1, Adadelta lr 0.02, 20 epochs, <= 1000 samples,
mini-batch 32, discount 0.9, acceptance probability exp(-gamma * (v - best) / best).
"""
import copy
import heapq
import json
import os

import numpy as np
import torch
import torch.nn as nn

from .utils import assert_print

global_walker_judger_model_path_prefix = "walker_judger_model_"
global_walker_judger_data_path_prefix = "walker_judger_data_"
global_performance_judger_path_prefix = "performance_judger_model_"
global_performance_data_path_prefix = "performance_judger_data_"


class Judger(nn.Module):
    def __init__(self, input_len, width, depth, output_len):
        super().__init__()
        assert_print(isinstance(width, int) and width > 0)
        assert_print(isinstance(depth, int) and depth > 1)
        layers = [("input", nn.Linear(input_len, width)), ("input_activate", nn.ReLU())]
        for count in range(depth - 2):
            layers.append(("hidden_{}".format(count), nn.Linear(width, width)))
            layers.append(("hidden_{}_activate".format(count), nn.ReLU()))
        layers.append(("output", nn.Linear(width, output_len)))
        self.net = nn.Sequential()
        for name, layer in layers:
            self.net.add_module(name, layer)

    def forward(self, inputs):
        return self.net(inputs)


def _minibatch_fit(params, samples, loss_of, lr, epochs=20, batch=32, on_epoch=None):
    """Shared training loop: accumulate the loss of `batch` samples, then step Adadelta."""
    optimizer = torch.optim.Adadelta(params, lr=lr)
    last = 0.0
    for ep in range(epochs):
        pending, total = None, 0.0
        for i, sample in enumerate(samples):
            term = loss_of(sample)
            pending = term if pending is None else pending + term
            total += float(term.detach())
            if (i + 1) % batch == 0:
                optimizer.zero_grad()
                pending.backward()
                optimizer.step()
                pending = None
        if pending is not None:
            optimizer.zero_grad()
            pending.backward()
            optimizer.step()
        last = total
        if on_epoch is not None:
            on_epoch(ep, total)
    return last


class Walker(nn.Module):
    def __init__(self, name, subspace, input_len):
        super().__init__()
        self.subspace = subspace
        self.pre_judger = Judger(input_len, 64, 4, self.subspace.num_direction)
        self.post_judger = Judger(input_len, 64, 4, self.subspace.num_direction)  # target net
        self.memory = []  # (pre_state, action, post_state, reward)
        self.mem_size = 0
        self.model_path = global_walker_judger_model_path_prefix + name + ".pkl"
        self.data_path = global_walker_judger_data_path_prefix + name + ".txt"

    def random_batch(self, batch_size):
        indices = np.random.randint(0, self.subspace.size, batch_size)
        return self._get_batch(indices), indices

    def _get_batch(self, indices):
        return [self.subspace.get_entity(int(i)) for i in indices]

    def walk(self, inputs, index_lst, trial, epsilon, gamma):
        """One epsilon-greedy step for each point; returns (new indices, chosen directions)."""
        q_values_lst = self.pre_judger(torch.FloatTensor(inputs)).detach()
        threshold = max(epsilon * np.exp(-trial * gamma), 0.1)
        new_indices, choices = [], []
        for i, q_values in enumerate(q_values_lst):
            if np.random.random() <= threshold:
                choice = int(np.random.randint(0, self.subspace.num_direction))
            else:
                choice = int(torch.argmax(q_values, dim=-1))
            direction = self.subspace.get_direction(choice)
            new_indices.append(self.subspace.next_entity(index_lst[i], direction))
            choices.append(choice)
        return new_indices, choices

    def full_walk(self, index):
        """A step in every direction of the sub-space."""
        moved = [self.subspace.next_entity(index, d) for d in self.subspace.directions]
        return moved, copy.deepcopy(self.subspace.directions)

    def add_data(self, pre_state, action, post_state, reward):
        self.memory.append((pre_state, action, post_state, reward))
        self.mem_size += 1

    def _action_index(self, action):
        if isinstance(action, (tuple, list)):
            return self.subspace.directions.index(tuple(action))
        return int(action)

    def train(self, lr=0.02, decay=0.9, save=True, verbose=True):
        np.random.shuffle(self.memory)
        samples = self.memory[:min(self.mem_size, 1000)]
        if verbose:
            print("train walker data size %d" % len(samples))
        if not samples:
            return

        def loss_of(sample):
            pre_state, action, post_state, reward = sample
            y = self.pre_judger(torch.FloatTensor(pre_state))[self._action_index(action)]
            nxt = self.post_judger(torch.FloatTensor(post_state)).detach()
            target = torch.max(nxt, dim=-1)[0] * decay + reward
            return torch.pow(y - target, 2)

        def on_epoch(ep, total):
            if save:
                self.save_model(self.model_path)
            if verbose:
                print("[cur/total]=[%d/%d] | loss=%f" % (ep + 1, 20, total))

        _minibatch_fit(self.pre_judger.parameters(), samples, loss_of, lr, on_epoch=on_epoch)
        if not save:
            self.post_judger.load_state_dict(self.pre_judger.state_dict())

    def save_model(self, model_path):
        self.post_judger.load_state_dict(self.pre_judger.state_dict())
        torch.save(self.pre_judger.state_dict(), model_path)

    def load_model(self, model_path):
        self.pre_judger.load_state_dict(torch.load(model_path))
        self.post_judger.load_state_dict(self.pre_judger.state_dict())

    def save_data(self, data_path):
        with open(data_path, "a") as fout:
            for data in self.memory:
                fout.write(json.dumps(data) + "\n")

    def load_data(self, data_path):
        with open(data_path, "r") as fin:
            for line in fin:
                self.memory.append(tuple(json.loads(line)))
                self.mem_size += 1

    def dump_data(self):
        self.save_data(self.data_path)

    def load_or_create_model(self):
        if os.path.exists(self.model_path):
            self.load_model(self.model_path)
        else:
            self.save_model(self.model_path)

    def prepare_data(self):
        if not os.path.exists(self.data_path):
            raise RuntimeError("Data file not found %s" % self.data_path)
        self.load_data(self.data_path)

    def clear_data(self):
        self.memory.clear()
        self.mem_size = 0


class MemEntity(object):
    def __init__(self, indices, value):
        self.indices = indices
        self.value = value

    def __lt__(self, other):
        return self.value < other.value


def rank_loss(y, t):
    assert len(y) == len(t)
    diff_t = torch.sign(t.reshape(-1, 1) - t.reshape(1, -1))
    diff_y = y.reshape(-1, 1) - y.reshape(1, -1)
    return torch.log(1 + torch.exp(-diff_t * diff_y)).sum()


class PerformanceModel(nn.Module):
    def __init__(self, input_len):
        super().__init__()
        self.input_len = input_len
        widths = [input_len, 32, 64, 128, 64, 16, 1]
        self.linears = nn.ModuleList(nn.Linear(a, b, bias=True) for a, b in zip(widths[:-1], widths[1:]))
        self.dropouts = nn.ModuleList(nn.Dropout(p=0.01) for _ in range(4))

    def forward(self, inputs):
        x = inputs
        for i, linear in enumerate(self.linears):
            x = linear(x)
            if i < len(self.dropouts):
                x = self.dropouts[i](x)
            x = torch.relu(x)
        return x


class WalkerGroup(object):
    def __init__(self, group_name, space, lr=0.02):
        self.space = space
        self.lr = lr
        self.walkers = {name: Walker(group_name + "_" + name, sub, self.space.dim) for name, sub in space.items()}
        self.memory = []
        self.mem_size = 0
        self.visit = set()
        self.performance_judger = PerformanceModel(max(self.space.dim, 1))
        self.perfromance_data = []
        self.model_path = global_performance_judger_path_prefix + group_name + ".pkl"
        self.data_path = global_performance_data_path_prefix + group_name + ".txt"

    # ---- sampling
    def forward(self, batch_size, policy="random"):
        assert_print(policy in ["random"])
        return {name: walker.random_batch(batch_size) for name, walker in self.walkers.items()}

    # ---- visited set and heap memory
    def ever_met(self, indices):
        return str(indices) in self.visit

    def _accept(self, value, gamma):
        best = self.top1_value()
        if not np.isfinite(best) or best <= 0:
            return True
        return np.random.random() <= np.exp(-gamma * (value - best) / best)

    def record(self, indices, value, random_reject=False, gamma=0.5):
        self.visit.add(str(indices))
        if random_reject and not self._accept(value, gamma):
            return
        heapq.heappush(self.memory, MemEntity(indices, value))
        self.mem_size += 1

    def has_more(self):
        return self.mem_size > 0

    def flatten(self, indices):
        flat = []
        for name, index in indices.items():
            flat.extend(self.walkers[name].subspace.get_entity(index))
        return flat

    def to_config(self, indices):
        """{type_key: [entity of each sub-space of that type, in insertion order]}."""
        config = {}
        for type_key, names in self.space.types.items():
            config[type_key] = [self.walkers[n].subspace.get_entity(indices[n]) for n in names if n in indices]
        return config

    def top_random(self, gamma=0.5, with_value=False):
        pick = self.memory[np.random.randint(0, len(self.memory))]
        if not self._accept(pick.value, gamma):
            pick = self.memory[0]
        return (pick.indices, pick.value) if with_value else pick.indices

    def topk(self, k, modify=False, with_value=False):
        k = min(k, self.mem_size)
        popped = [heapq.heappop(self.memory) for _ in range(k)]
        self.mem_size -= k
        if not modify:
            for item in popped:
                heapq.heappush(self.memory, item)
            self.mem_size += k
        if with_value:
            return [(x.indices, x.value) for x in popped]
        return [x.indices for x in popped]

    def top1(self):
        return self.memory[0].indices if self.mem_size > 0 else {}

    def top1_value(self):
        return self.memory[0].value if self.mem_size > 0 else float("inf")

    def pop_top(self):
        if self.mem_size > 0:
            self.mem_size -= 1
            return heapq.heappop(self.memory)
        return MemEntity({}, float("inf"))

    # ---- moves
    def walk(self, indices_value_lst, trial, epsilon=0.8, gamma=0.01):
        """Every point takes one step in every sub-space; only unseen results are returned."""
        indices_lst = [x[0] for x in indices_value_lst]
        value_lst = [x[1] for x in indices_value_lst]
        flattened = [self.flatten(indices) for indices in indices_lst]
        from_lst, next_lst, action_lst = [], [], []
        if not indices_lst:
            return from_lst, next_lst, action_lst
        for name, walker in self.walkers.items():
            cur = [indices[name] for indices in indices_lst]
            moved, choices = walker.walk(flattened, cur, trial, epsilon, gamma)
            for i, (new_index, choice) in enumerate(zip(moved, choices)):
                nxt = copy.deepcopy(indices_lst[i])
                nxt[name] = new_index
                if not self.ever_met(nxt):
                    from_lst.append((indices_lst[i], value_lst[i]))
                    next_lst.append(nxt)
                    action_lst.append((name, choice))
        return from_lst, next_lst, action_lst

    def full_walk(self, indices, no_repeat=True):
        next_lst, action_lst = [], []
        for name, index in indices.items():
            moved, directions = self.walkers[name].full_walk(index)
            for new_index, direction in zip(moved, directions):
                nxt = copy.deepcopy(indices)
                nxt[name] = new_index
                if no_repeat and self.ever_met(nxt):
                    continue
                next_lst.append(nxt)
                action_lst.append((name, direction))
        return next_lst, action_lst

    # ---- learning
    def add_data(self, name, pre_state, action, post_state, reward):
        self.walkers[name].add_data(self.flatten(pre_state), action, self.flatten(post_state), float(reward))

    def train_walkers(self, save=True, verbose=True):
        for walker in self.walkers.values():
            walker.train(lr=self.lr, save=save, verbose=verbose)

    def add_perf_data(self, indices_lst, performance_lst):
        self.perfromance_data.append(([self.flatten(ind) for ind in indices_lst], list(performance_lst)))

    def train_on_perf(self, save=True, verbose=True):
        np.random.shuffle(self.perfromance_data)
        samples = [d for d in self.perfromance_data[:1000] if len(d[0]) > 0]
        if verbose:
            print("train data size is %d" % len(samples))
        if not samples:
            return

        def loss_of(sample):
            x, t = sample
            t = [min(v, 1e6) for v in t]  # failed measurements are inf
            y = self.performance_judger(torch.FloatTensor(x)).reshape(-1)
            return rank_loss(y, torch.FloatTensor(t))

        def on_epoch(ep, total):
            if save:
                self.save_performance_judger(self.model_path)
            if verbose:
                print("[cur/total]=[%d/%d] | loss=%f" % (ep + 1, 20, total))

        _minibatch_fit(self.performance_judger.parameters(), samples, loss_of, self.lr, on_epoch=on_epoch)

    def test_accuracy(self):
        samples = [d for d in self.perfromance_data[:1000] if len(d[0]) > 0]
        loss = 0.0
        for x, t in samples:
            y = self.performance_judger(torch.FloatTensor(x)).reshape(-1)
            loss += float(rank_loss(y, torch.FloatTensor([min(v, 1e6) for v in t])).detach())
        return loss / max(len(samples), 1)

    def query_performance(self, indices_lst):
        inputs = [self.flatten(ind) for ind in indices_lst]
        if not inputs:
            return []
        self.performance_judger.eval()
        out = self.performance_judger(torch.FloatTensor(inputs)).reshape(-1).detach().tolist()
        self.performance_judger.train()
        return out

    # ---- persistence
    def load_performance_judger(self, model_path):
        self.performance_judger.load_state_dict(torch.load(model_path))

    def save_performance_judger(self, model_path):
        torch.save(self.performance_judger.state_dict(), model_path)

    def dump_performance_data(self, data_path):
        with open(data_path, "a") as fout:
            for data in self.perfromance_data:
                fout.write(json.dumps(data) + "\n")

    def load_performance_data(self, data_path):
        with open(data_path, "r") as fin:
            for line in fin:
                self.perfromance_data.append(tuple(json.loads(line)))

    def dump_data(self):
        self.dump_performance_data(self.data_path)
        for walker in self.walkers.values():
            walker.dump_data()

    def load_walker_model(self):
        for walker in self.walkers.values():
            walker.load_or_create_model()

    def load_walker_data(self):
        for walker in self.walkers.values():
            walker.prepare_data()

    def prepare_performance_data(self):
        if not os.path.exists(self.data_path):
            raise RuntimeError("Performance data file not found %s" % self.data_path)
        self.load_performance_data(self.data_path)

    def load_or_create_model(self):
        if os.path.exists(self.model_path):
            self.load_performance_judger(self.model_path)
        else:
            self.save_performance_judger(self.model_path)

    def clear_performance_data(self):
        self.perfromance_data.clear()

    def clear_walker_data(self):
        for walker in self.walkers.values():
            walker.clear_data()

    def clear_data(self):
        self.clear_performance_data()
        self.clear_walker_data()
