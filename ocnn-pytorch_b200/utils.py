"""Small helpers with the names and behaviour of the reference's ocnn/utils.py."""
import math

import torch


def resize_with_last_val(list_in: list, num: int = 3):
  r''' Pads :attr:`list_in` to :attr:`num` entries with its last value (utils.py:169-179). '''
  assert (type(list_in) is list and len(list_in) < num + 1)
  list_out = list(list_in)
  for _ in range(len(list_out), num):
    list_out.append(list_out[-1])
  return list_out


def list2str(list_in: list):
  r''' ``[3, 3, 3] -> '333'`` (utils.py:182-187). '''
  return ''.join(str(x) for x in list_in)


def xavier_uniform_(weights: torch.Tensor):
  r''' Xavier-uniform initialisation for weights of shape ``(kdim, in_c, out_c)``:
  ``fan_in = kdim * in_c``, ``fan_out = kdim * out_c`` (utils.py:150-166). '''
  shape = weights.shape
  fan_in = shape[0] * shape[1]
  fan_out = shape[0] * shape[2]
  std = math.sqrt(2.0 / float(fan_in + fan_out))
  a = math.sqrt(3.0) * std
  torch.nn.init.uniform_(weights, -a, a)


def cumsum(data: torch.Tensor, dim: int, exclusive: bool = False):
  r''' :func:`torch.cumsum` with an optional leading zero (utils.py:77-96). '''
  out = torch.cumsum(data, dim)
  if exclusive:
    size = list(data.size())
    size[dim] = 1
    out = torch.cat([out.new_zeros(size), out], dim)
  return out
