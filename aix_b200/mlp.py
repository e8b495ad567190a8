"""The MLP training configuration: 4 Linear layers 1024 -> 4096 -> 4096 -> 4096 -> 1024 with tanh between them,
float32, Xavier-uniform weights, MSE loss, Adam(1e-3, 0.9, 0.999); one step = forward + backward + (gradient
all-reduce over the ranks) + optimizer step, issued through the mirrored front end (aix_b200/frontend.py)."""
import numpy as np

from . import _capi as C
from .frontend import (Adam, GradientExchange, Linear, MSELoss, Sequential, ShardedAdam, ShardedGradientExchange, Tanh, Tensor,
                       all_reduce_gradients)
from .tensor import TensorValue

DEFAULT_DIMS = (1024, 4096, 4096, 4096, 1024)


def xavier_parameters(dims, seed=0):
    """U(-sqrt(6/(in+out)), +sqrt(6/(in+out))) weights and zero biases, identical on every rank."""
    rng = np.random.default_rng(seed)
    weights, biases = [], []
    for fan_in, fan_out in zip(dims[:-1], dims[1:]):
        bound = np.sqrt(6.0 / (fan_in + fan_out))
        weights.append(rng.uniform(-bound, bound, (fan_in, fan_out)).astype(np.float32))
        biases.append(np.zeros((1, fan_out), dtype=np.float32))
    return weights, biases


def synthetic_batch(dims, batch, rank=0, seed=0):
    """Inputs and targets ~ N(0,1); rank r draws from the seed-0 stream offset by r."""
    rng = np.random.default_rng([seed, rank])
    x = rng.normal(0, 1, (batch, dims[0])).astype(np.float32)
    y = rng.normal(0, 1, (batch, dims[-1])).astype(np.float32)
    return x, y


class MlpTrainer:
    def __init__(self, device, dims=DEFAULT_DIMS, batch=4096, rank=0, world_size=1, lr=1e-3, seed=0, weights=None, biases=None,
                 overlap=True, data=None, sharded=False, deferred=False, early=False):
        self.device, self.dims, self.world_size = device, tuple(dims), world_size
        if weights is None:
            weights, biases = xavier_parameters(dims, seed)
        layers = []
        for i, (w, b) in enumerate(zip(weights, biases)):
            layers.append(Linear(w, b, device))
            if i + 1 < len(weights):
                layers.append(Tanh())
        self.model = Sequential(*layers)
        x, y = data if data is not None else synthetic_batch(dims, batch, rank, seed)
        batch = x.shape[0]
        self.x = Tensor(TensorValue.from_numpy(x, device))
        self.y = Tensor(TensorValue.from_numpy(y, device))
        # sharded=True: reduce-scatter the gradients, update 1/world_size of every parameter (and keep that share of the
        # Adam state) per rank, all-gather the parameters; needs the overlapped exchange. deferred / early move the updates
        # of the late / early layers into the next forward pass / into backward() (ShardedAdam.attach_model,
        # ShardedGradientExchange.attach). Measured on 8 B200 they are within 1 % of the plain sharded form (all with the
        # all-gathers on a communicator of their own, the device's default), so the plain form is the default.
        sharded = sharded and overlap and world_size > 1
        params = self.model.parameters()
        self.optimizer = ShardedAdam(params, rank, world_size, lr=lr) if sharded else Adam(params, lr=lr)   # after the parameters live on the device
        if sharded and deferred:
            self.optimizer.attach_model(self.model)         # updates applied layer by layer inside the next forward pass
        self.loss_fn = MSELoss()
        # overlap=True: each gradient's collective starts inside backward(); False: all of them after it
        exchange_type = ShardedGradientExchange if sharded else GradientExchange
        self.exchange = exchange_type(device, params, world_size) if overlap and world_size > 1 else None
        if self.exchange is not None:
            # early: the first layers' updates and all-gathers move into backward() (valid for this feed-forward stack)
            if sharded and deferred and early:
                self.exchange.attach(self.optimizer, early=True)
            else:
                self.exchange.attach(self.optimizer)
        self.flops_per_step = 2.0 * batch * sum(a * b for a, b in zip(dims[:-1], dims[1:])) * 3 \
            - 2.0 * batch * dims[0] * dims[1]                        # forward + dW + dX (no dX for the first layer)

    def set_batch(self, x_ptr, y_ptr):
        """Copies a new batch from (pinned) host memory into the resident input tensors."""
        self.device.copy(x_ptr, C.F32, self.x.value.storage.data, C.F32, self.x.value.size)
        self.device.copy(y_ptr, C.F32, self.y.value.storage.data, C.F32, self.y.value.size)

    def step(self) -> Tensor:
        pred = self.model.forward(self.x)
        loss = self.loss_fn(pred, self.y)
        self.optimizer.zeroGrad()
        loss.backward()
        if self.exchange is not None:
            self.exchange.finish()
        else:
            all_reduce_gradients(self.device, self.model.parameters(), self.world_size)
        self.optimizer.step()
        return loss

    def parameters_numpy(self):
        if hasattr(self.optimizer, "finish"):
            self.optimizer.finish()                         # a deferred optimizer may still owe the last step's updates
        return [p.value.numpy() for p in self.model.parameters()]
