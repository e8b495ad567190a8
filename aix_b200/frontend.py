"""Host-side mirror of the callers of the device on the training path: aix::Tensor with autograd, nn::Linear / Tanh /
Sequential / MSELoss and optim::Adam / SGD.

Only what the MLP training configuration needs is mirrored, and it is mirrored literally: every method issues the
device calls of the reference method it cites, in the same order, so that a training step drives the device with
the op stream of the reference front end (4 Linear layers: 17 forward ops, 8 zero-fills, 39 backward ops, 22 ops per
parameter in Adam). Nothing here computes; all arithmetic happens in device calls.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import numpy as np

from . import _capi as C
from .tensor import _TO_FLOAT, TensorValue, promote


class TensorNode:
    """aix::TensorNode (aixCore.hpp:1790-1857)."""

    def __init__(self, value: TensorValue, requireGrad: bool = False):
        self.value = value
        self.requireGrad = requireGrad
        self.retainGrad = False
        self.isLeaf = True
        self.inputs: List["TensorNode"] = []
        self.backwardFunc: Callable = defaultBackward
        self._grad: Optional[TensorValue] = None
        self.gradReadyHook: Optional[Callable] = None   # no counterpart in the reference; see GradientExchange

    def grad(self) -> TensorValue:
        if self._grad is None:
            self._grad = TensorValue.empty(self.value.shape, self.value.device, self.value.dtype)
            self._grad.fill(0)
        return self._grad

    def backward(self, seed: TensorValue):
        if _readyNodes:
            _callReadyHooks()
        if self.retainGrad:
            g = self.grad()
            g += seed
        if self.requireGrad or self.retainGrad:
            self.backwardFunc(self, seed)

    def setBackward(self, inputs, func):
        if self.requireGrad or self.retainGrad:
            self.inputs = list(inputs)
            self.backwardFunc = func


def _wants(node: TensorNode) -> bool:
    return node.requireGrad or node.retainGrad


# ---- backward functions (aixCore.hpp:2014-2247) ---------------------------------------------------------------------
def defaultBackward(node: TensorNode, seed: TensorValue):
    if node.requireGrad and not node.retainGrad:
        g = node.grad()
        g += seed                                  # in-place Device::add into the gradient buffer
        if node.gradReadyHook is not None:
            _readyNodes.append(node)


# Gradient-ready hooks (no counterpart in the reference) are not called from inside defaultBackward but at the next step of the
# backward pass - the next TensorNode.backward call, or the end of Tensor.backward. By then the caller has dropped the
# temporary it accumulated (`W.backward(x^T . G)`), so a device that holds the product back can still write it straight into
# the gradient buffer; a hook called at once would start a collective, which launches everything recorded, while the
# temporary is still referenced.
_readyNodes: List[TensorNode] = []


def _callReadyHooks():
    while _readyNodes:
        node = _readyNodes.pop(0)
        if node.gradReadyHook is not None:
            node.gradReadyHook(node)


def broadcastBackwardFunc(node, seed):
    if node.inputs:
        node.inputs[0].backward(seed.reduceTo(node.inputs[0].value.shape))


def addBackwardFunc(node, seed):
    if len(node.inputs) < 2: return
    if node.inputs[0] is node.inputs[1]:
        node.inputs[0].backward(seed + seed)
        return
    if _wants(node.inputs[0]): node.inputs[0].backward(seed)
    if _wants(node.inputs[1]): node.inputs[1].backward(seed)


def subBackwardFunc(node, seed):
    if len(node.inputs) < 2 or node.inputs[0] is node.inputs[1]: return
    if _wants(node.inputs[0]): node.inputs[0].backward(seed)
    if _wants(node.inputs[1]): node.inputs[1].backward(-seed)


def mulBackwardFunc(node, seed):
    if len(node.inputs) < 2: return
    if node.inputs[0] is node.inputs[1]:
        grad = node.inputs[0].value * seed
        node.inputs[0].backward(grad + grad)
        return
    if _wants(node.inputs[0]): node.inputs[0].backward(node.inputs[1].value * seed)
    if _wants(node.inputs[1]): node.inputs[1].backward(node.inputs[0].value * seed)


def divBackwardFunc(node, seed):
    if len(node.inputs) < 2: return
    if _wants(node.inputs[0]): node.inputs[0].backward(seed / node.inputs[1].value)
    if _wants(node.inputs[1]):
        b = node.inputs[1].value
        node.inputs[1].backward(-node.inputs[0].value * seed / (b * b))


def unaryBackwardFunc(node, seed):
    if node.inputs: node.inputs[0].backward(-seed)


def tanhBackwardFunc(node, seed):
    if node.inputs:
        t = node.value
        node.inputs[0].backward((1.0 - t * t) * seed)


def sinBackwardFunc(node, seed):
    if node.inputs: node.inputs[0].backward(node.inputs[0].value.cos() * seed)       # aixCore.hpp:2123-2129


def cosBackwardFunc(node, seed):
    if node.inputs: node.inputs[0].backward(-node.inputs[0].value.sin() * seed)      # aixCore.hpp:2131-2137


def matmulBackwardFunc(node, seed):
    if len(node.inputs) < 2: return
    a, b = node.inputs
    if a is b:
        xT = a.value.transpose(0, 1)
        a.backward(seed.matmul(xT) + xT.matmul(seed))
        return
    if _wants(a): a.backward(seed.matmul(b.value.transpose(0, 1)))
    if _wants(b): b.backward(a.value.transpose(0, 1).matmul(seed))


def sumBackwardFunc(node, seed):
    if node.inputs: node.inputs[0].backward(seed.broadcastTo(node.inputs[0].value.shape))


class Tensor:
    """aix::Tensor (aixCore.hpp:1879-2893), the subset on the MLP training path."""

    def __init__(self, value: TensorValue, requireGrad: bool = False):
        self.node = TensorNode(value, requireGrad)

    @staticmethod
    def _result(value: TensorValue, anyRequiresGrad: bool, anyNonLeaf: bool = False) -> "Tensor":
        t = Tensor(value, anyRequiresGrad)           # makeResult (aixCore.hpp:2788-2796)
        t.node.isLeaf = not anyRequiresGrad and not anyNonLeaf
        return t

    # accessors
    @property
    def value(self) -> TensorValue: return self.node.value
    @property
    def shape(self): return self.node.value.shape
    @property
    def dtype(self): return self.node.value.dtype
    @property
    def device(self): return self.node.value.device
    def grad(self) -> TensorValue: return self.node.grad()
    def isRequireGrad(self) -> bool: return self.node.requireGrad
    def zeroGrad(self): self.node.grad().fill(0)

    def backward(self):
        """aixCore.hpp:1921-1931: seed of ones in the tensor's own shape."""
        v = self.node.value
        seed = TensorValue.full(1, v.shape, v.device, v.dtype)
        self.node.backward(seed)
        _callReadyHooks()

    # views / conversions
    def broadcastTo(self, shape) -> "Tensor":
        if tuple(shape) == tuple(self.shape): return self
        r = Tensor._result(self.value.broadcastTo(shape), self.isRequireGrad())
        r.node.setBackward([self.node], broadcastBackwardFunc)
        return r

    def _binary(self, other, op: str, backward) -> "Tensor":
        if not isinstance(other, Tensor):
            one = TensorValue.full(float(other), (), self.device, _TO_FLOAT[self.dtype])
            other = Tensor(one).broadcastTo(self.shape)         # aixCore.hpp:2384-2406
        dtype = promote(self.dtype, other.dtype)
        shape = self.shape if tuple(self.shape) == tuple(other.shape) else tuple(np.broadcast_shapes(self.shape, other.shape))
        lhs, rhs = self.broadcastTo(shape), other.broadcastTo(shape)
        assert lhs.dtype == dtype and rhs.dtype == dtype, "mixed element types are not on the mirrored path"
        value = getattr(lhs.value, op)(rhs.value)
        r = Tensor._result(value, self.isRequireGrad() or other.isRequireGrad(), not lhs.node.isLeaf or not rhs.node.isLeaf)
        r.node.setBackward([lhs.node, rhs.node], backward)
        return r

    def __add__(self, o): return self._binary(o, "__add__", addBackwardFunc)
    def __sub__(self, o): return self._binary(o, "__sub__", subBackwardFunc)
    def __mul__(self, o): return self._binary(o, "__mul__", mulBackwardFunc)
    def __truediv__(self, o): return self._binary(o, "__truediv__", divBackwardFunc)

    def __neg__(self) -> "Tensor":
        r = Tensor._result(-self.value, self.isRequireGrad())
        r.node.setBackward([self.node], unaryBackwardFunc)
        return r

    def tanh(self) -> "Tensor":
        r = Tensor._result(self.value.tanh(), self.isRequireGrad())
        r.node.setBackward([self.node], tanhBackwardFunc)
        return r

    def sin(self) -> "Tensor":
        r = Tensor._result(self.value.sin(), self.isRequireGrad())
        r.node.setBackward([self.node], sinBackwardFunc)
        return r

    def cos(self) -> "Tensor":
        r = Tensor._result(self.value.cos(), self.isRequireGrad())
        r.node.setBackward([self.node], cosBackwardFunc)
        return r

    def matmul(self, other: "Tensor") -> "Tensor":
        r = Tensor._result(self.value.matmul(other.value), self.isRequireGrad() or other.isRequireGrad(),
                           not self.node.isLeaf or not other.node.isLeaf)
        r.node.setBackward([self.node, other.node], matmulBackwardFunc)
        return r

    def sum(self) -> "Tensor":
        r = Tensor._result(self.value.sum(), self.isRequireGrad())
        r.node.setBackward([self.node], sumBackwardFunc)
        return r

    def mean(self) -> "Tensor":
        return self.sum() / float(self.value.size)             # aixCore.hpp:2498-2501


# ---- nn (aixNeuralNetwork.hpp) ---------------------------------------------------------------------------------------
class Linear:
    """nn::Linear (aixNeuralNetwork.hpp:132-157): W is {in, out}, b is {1, out}, forward = matmul(x, W) + b."""

    def __init__(self, weight: np.ndarray, bias: np.ndarray, device, dtype: int = C.F32):
        self.w = Tensor(TensorValue.from_numpy(weight, device, dtype), requireGrad=True)
        self.b = Tensor(TensorValue.from_numpy(bias.reshape(1, -1), device, dtype), requireGrad=True)

    def parameters(self): return [self.w, self.b]
    def forward(self, x: Tensor) -> Tensor: return x.matmul(self.w) + self.b


class Tanh:
    def parameters(self): return []
    def forward(self, x: Tensor) -> Tensor: return x.tanh()


class Sequential:
    def __init__(self, *modules):
        self.modules = list(modules)
        self.beforeModule: Optional[Callable] = None    # no counterpart in the reference; see ShardedAdam.attach_model

    def parameters(self): return [p for m in self.modules for p in m.parameters()]

    def forward(self, x: Tensor) -> Tensor:
        for index, m in enumerate(self.modules):
            if self.beforeModule is not None:
                self.beforeModule(index)
            x = m.forward(x)
        return x


class MSELoss:
    """nn::MSELoss (aixNeuralNetwork.hpp:222-231): mean(diff * diff)."""

    def __call__(self, predictions: Tensor, targets: Tensor) -> Tensor:
        diff = predictions - targets
        return (diff * diff).mean()


# ---- optim (aixOptimizer.hpp) ------------------------------------------------------------------------------------------
class SGD:
    def __init__(self, parameters: Sequence[Tensor], lr: float = 0.01):
        self.parameters, self.lr = list(parameters), lr

    def zeroGrad(self):
        for p in self.parameters: p.zeroGrad()

    def step(self):                                  # aixOptimizer.hpp:76-86
        for p in self.parameters:
            if p.isRequireGrad():
                v = p.value
                v -= p.grad() * self.lr


class Adam:
    """optim::Adam (aixOptimizer.hpp:93-159); state tensors live on the parameters' device."""

    def __init__(self, parameters: Sequence[Tensor], lr=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.parameters = list(parameters)
        self.lr, self.beta1, self.beta2, self.epsilon = lr, beta1, beta2, epsilon
        self.timestep = 0
        self.beforeParameter: Optional[Callable] = None     # no counterpart in the reference; see GradientExchange.attach
        self.m = [TensorValue.full(0.0, p.shape, p.device, C.F32) for p in self.parameters]
        self.v = [TensorValue.full(0.0, p.shape, p.device, C.F32) for p in self.parameters]

    def zeroGrad(self):
        for p in self.parameters: p.zeroGrad()

    def step(self):
        self.timestep += 1
        # The reference's members are floats and its expressions are evaluated in double, then narrowed:
        # float(1.0 - m_beta1), float(1.0 - std::pow(m_beta1, m_timestep)) (aixOptimizer.hpp:124-133).
        b1, b2 = float(np.float32(self.beta1)), float(np.float32(self.beta2))
        narrow = lambda x: float(np.float32(x))
        for i, p in enumerate(self.parameters):
            if not p.isRequireGrad():
                continue
            if self.beforeParameter is not None:
                self.beforeParameter(p)
            g = p.grad().to(C.F32)
            self.m[i] = self.beta1 * self.m[i] + narrow(1.0 - b1) * g
            self.v[i] = self.beta2 * self.v[i] + narrow(1.0 - b2) * g * g
            mHat = self.m[i] / narrow(1.0 - math.pow(b1, self.timestep))
            vHat = self.v[i] / narrow(1.0 - math.pow(b2, self.timestep))
            value = p.value
            value -= (self.lr * mHat / (vHat.sqrt() + self.epsilon)).to(p.dtype)


def all_reduce_gradients(device, parameters: Sequence[Tensor], world_size: int):
    """Data-parallel exchange between backward() and step(): sums every gradient over the ranks and divides by the
    number of ranks, so that each rank holds the gradient of the mean loss over the global batch. The reference has no
    such hook; gradients are plain tensor values reachable through Tensor::grad() (aixCore.hpp:1946-1956)."""
    if world_size <= 1:
        return
    for p in parameters:
        g = p.grad()
        device.allReduce(g.storage.data, g.size, g.dtype, 1.0 / world_size)


class GradientExchange:
    """The same exchange, overlapped with the rest of backward() and with the optimizer step: once a parameter's
    gradient has been accumulated (defaultBackward, aixCore.hpp:2014-2021; the hook runs at the backward pass's next
    step, see _callReadyHooks) its all-reduce starts on the device's side stream, so that the collectives of some layers run under the matmuls of the others. `attach(optimizer)` makes the
    optimizer join, before it starts on a parameter, only that parameter's collective: the front end produces the
    weight gradients first-layer-first, so the largest exchanges are the last to start, and Adam already runs on the
    first parameters while they finish. Without an attached optimizer, `finish()` joins everything at once; it goes
    between backward() and step() either way. The reference would need one hook call at the end of defaultBackward
    and one at the top of the optimizer's per-parameter loop.

    The device itself orders any op that touches a gradient after that gradient's collective, so a forgotten join
    cannot race; joining explicitly at a parameter boundary keeps each parameter's recorded ops in one kernel (a join
    in the middle of `beta1 * m + (1 - beta1) * g` would cut the expression in two launches and, with FMA contraction
    allowed, change last bits relative to the blocking form).

    Valid when every parameter receives exactly one gradient contribution per backward pass (true for a feed-forward
    stack); a second contribution to a gradient already in flight raises instead of racing with the collective."""

    def __init__(self, device, parameters: Sequence[Tensor], world_size: int):
        self.device, self.world_size = device, world_size
        self.parameters = list(parameters)
        self._inFlight = set()
        if world_size > 1:
            for p in self.parameters:
                p.node.gradReadyHook = self._ready

    def _ready(self, node: TensorNode):
        if id(node) in self._inFlight:
            raise RuntimeError("GradientExchange: a parameter received a second gradient contribution while its "
                               "all-reduce was in flight; use all_reduce_gradients for this model")
        self._inFlight.add(id(node))
        g = node.grad()
        self.device.allReduceAsync(g.storage.data, g.size, g.dtype, 1.0 / self.world_size)

    def attach(self, optimizer):
        if self.world_size > 1:
            optimizer.beforeParameter = self._join
            self._attached = True

    def _join(self, p: "Tensor"):
        g = p.grad()
        self.device.commWaitFor(g.storage.data, g.size * C.DTYPE_SIZES[g.dtype])

    def finish(self):
        if self.world_size > 1 and not getattr(self, "_attached", False):
            self.device.commWait()
        self._inFlight.clear()

    def detach(self):
        for p in self.parameters:
            p.node.gradReadyHook = None


def global_mean(value: TensorValue, world_size: int) -> TensorValue:
    """Mean over a tensor whose rows are split across `world_size` ranks (equal shards): the local `sum()` - folded into
    the producing kernel when that is still pending - one scalar all-reduce that averages the partial sums over the
    ranks, and the reference's `sum() / size` division (aixCore.hpp:2498-2501) by the LOCAL size. Row-wise results of a
    row-sharded tensor need no exchange at all."""
    total = value.sum()
    if world_size > 1:
        value.device.allReduce(total.storage.data, 1, total.dtype, 1.0 / world_size)
    return total / float(value.size)


def _flat_slice(t: TensorValue, rank: int, world_size: int) -> TensorValue:
    """Slice `rank` of `world_size` of a dense tensor, as a 1-D view of its storage."""
    n = t.size // world_size
    return TensorValue(t.storage, (n,), (1,), t.offset + rank * n, t.dtype, t.device)


class ShardedGradientExchange(GradientExchange):
    """Gradient exchange of the sharded optimizer: a reduce-scatter instead of an all-reduce, started from the same
    gradient-ready hook. Afterwards rank r holds the averaged gradient only in slice r of every gradient buffer, which
    is all ShardedAdam reads. Parameters whose size is not a multiple of the number of ranks keep the all-reduce."""

    def _ready(self, node: TensorNode):
        if id(node) in self._inFlight:
            raise RuntimeError("GradientExchange: a parameter received a second gradient contribution while its "
                               "collective was in flight; use all_reduce_gradients for this model")
        self._inFlight.add(id(node))
        g = node.grad()
        if g.size % self.world_size == 0:
            self.device.reduceScatterAsync(g.storage.data, g.size, g.dtype, 1.0 / self.world_size)
        else:
            self.device.allReduceAsync(g.storage.data, g.size, g.dtype, 1.0 / self.world_size)
        # Early updates (attach(optimizer, early=True)): the parameter whose collective was started two gradients ago has had
        # a whole weight-gradient matmul to finish it; its slice is updated and its all-gather started now, inside backward().
        early = getattr(self, "_early", None)
        if early is not None:
            self._order.append(early["index_of"].get(id(node)))
            if len(self._order) >= 3 and self._order[-3] in early["allowed"]:
                early["optimizer"].update_early(self._order[-3])

    def attach(self, optimizer, early: bool = False):
        """early=True (needs a ShardedAdam with a model attached): parameters of the modules the optimizer would update at
        once in step() are instead updated inside backward(), two gradient-ready hooks after their own - their
        reduce-scatter has finished under the matmul in between, and their all-gather then runs under the remaining
        weight-gradient matmuls instead of after them. ONLY valid when no parameter value is read by backward() after the
        first gradient is final: true for a feed-forward stack under the reference's recursion order (every dX is
        computed on the way down, before any dW, aixCore.hpp:2192-2207)."""
        super().attach(optimizer)
        if early and self.world_size > 1 and hasattr(optimizer, "_owners"):
            allowed = {i for j in optimizer._with_params[:optimizer._eager] for i in optimizer._owners[j]}
            self._early = {"optimizer": optimizer, "allowed": allowed, "index_of": {id(p.node): i for i, p in enumerate(optimizer.parameters)}}
            self._order = []

    def finish(self):
        super().finish()
        if getattr(self, "_early", None) is not None:
            self._order = []


class ShardedAdam(Adam):
    """optim::Adam (aixOptimizer.hpp:93-159) with its work and its state split over the data-parallel ranks: rank r keeps
    the moments of slice r of every parameter only, updates that slice from slice r of the reduce-scattered gradient
    with exactly the reference's expression sequence, and an all-gather hands every rank the other slices. The
    all-gather runs on the device's side stream; the device orders the first later use of the parameter (the next
    forward pass) after it. Elementwise the update is the reference's, so the parameters equal those of the unsharded
    optimizer given the same averaged gradients. A parameter whose size is not a multiple of the number of ranks is
    updated in full on every rank (its gradient was all-reduced)."""

    def __init__(self, parameters: Sequence[Tensor], rank: int, world_size: int, lr=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.parameters = list(parameters)
        self.lr, self.beta1, self.beta2, self.epsilon = lr, beta1, beta2, epsilon
        self.timestep = 0
        self.rank, self.world_size = rank, world_size
        self.beforeParameter: Optional[Callable] = None
        self.sharded = [world_size > 1 and p.value.size % world_size == 0 and p.value.isContiguous() for p in self.parameters]
        shape = lambda p, s: (p.value.size // world_size,) if s else p.shape
        self.m = [TensorValue.full(0.0, shape(p, s), p.device, C.F32) for p, s in zip(self.parameters, self.sharded)]
        self.v = [TensorValue.full(0.0, shape(p, s), p.device, C.F32) for p, s in zip(self.parameters, self.sharded)]

    def attach_model(self, model: "Sequential", lookahead: int = 1, eager_modules: Optional[int] = None):
        """Deferred form. The front end finishes the weight gradients first-layer-first, so the reduce-scatters of the LAST
        layers are still running when backward() returns; issued eagerly, their updates hold up the in-order stream - and
        the next forward pass behind them. With a model attached, `step()` updates only the first `eager_modules`
        parametrised modules at once (default: the first half - their gradients arrived long ago, and their all-gathers
        then run under the rest of step()); the others are noted as due and updated when the next forward pass reaches
        the module `lookahead` parametrised modules before their own, so that the first layers of that pass run under the
        late collectives and each late layer's update and all-gather run under the layer before it. Every parameter is
        still updated before its next use; `finish()` applies whatever is outstanding (before the host reads
        parameters)."""
        self._owners = []                                   # per module: indices of its parameters in self.parameters
        index_of = {id(p.node): i for i, p in enumerate(self.parameters)}
        for m in model.modules:
            self._owners.append([index_of[id(p.node)] for p in m.parameters() if id(p.node) in index_of])
        self._with_params = [j for j, own in enumerate(self._owners) if own]
        self._lookahead = lookahead
        self._eager = len(self._with_params) // 2 if eager_modules is None else eager_modules
        self._due = set()
        model.beforeModule = self._before_module

    def _before_module(self, module_index: int):
        if not self._due or module_index not in self._with_params:
            return
        at = self._with_params.index(module_index)
        for j in self._with_params[:at + 1 + self._lookahead]:
            for i in self._owners[j]:
                if i in self._due:
                    self._due.discard(i)
                    self._update(i)

    def finish(self):
        for i in sorted(getattr(self, "_due", ())):
            self._update(i)
        if hasattr(self, "_due"):
            self._due.clear()

    def update_early(self, i: int):
        """Applies parameter i's update of the step that the next step() call counts, ahead of that call (from a
        gradient-ready hook inside backward(): ShardedGradientExchange.attach(early=True))."""
        done = self.__dict__.setdefault("_done_early", set())
        if i not in done and self.parameters[i].isRequireGrad():
            done.add(i)
            self._update(i, self.timestep + 1)

    def step(self):
        self.finish()                                       # nothing of the previous step may be left when the gradients change
        self.timestep += 1
        done = self.__dict__.setdefault("_done_early", set())
        if hasattr(self, "_owners"):
            self._due = {i for i, p in enumerate(self.parameters) if p.isRequireGrad() and i not in done}
            done.clear()
            for j in self._with_params[:self._eager]:
                for i in self._owners[j]:
                    if i in self._due:
                        self._due.discard(i)
                        self._update(i)
            return
        for i, p in enumerate(self.parameters):
            if p.isRequireGrad() and i not in done:
                self._update(i)
        done.clear()

    def _update(self, i: int, timestep: Optional[int] = None):
        timestep = self.timestep if timestep is None else timestep
        p = self.parameters[i]
        b1, b2 = float(np.float32(self.beta1)), float(np.float32(self.beta2))
        narrow = lambda x: float(np.float32(x))
        if self.beforeParameter is not None:
            self.beforeParameter(p)
        value, grad = p.value, p.grad()
        if self.sharded[i]:
            value, grad = _flat_slice(value, self.rank, self.world_size), _flat_slice(grad, self.rank, self.world_size)
        g = grad.to(C.F32)
        self.m[i] = self.beta1 * self.m[i] + narrow(1.0 - b1) * g
        self.v[i] = self.beta2 * self.v[i] + narrow(1.0 - b2) * g * g
        mHat = self.m[i] / narrow(1.0 - math.pow(b1, timestep))
        vHat = self.v[i] / narrow(1.0 - math.pow(b2, timestep))
        value -= (self.lr * mHat / (vHat.sqrt() + self.epsilon)).to(p.dtype)
        if self.sharded[i]:
            whole = p.value
            whole.device.allGatherAsync(whole.storage.data, whole.size, whole.dtype)
