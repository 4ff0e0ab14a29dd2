"""(batch, head) sharding across the GPUs of one box.

Every (batch, head) pair of every case is an independent unit (the reference treats B and H as
pure grid axes, lib/Dialect/Asuka/Transforms/Parallelize.cpp:38-48), so the units are split into
contiguous ranges, one per rank, and no collective is needed on the data path.
"""


def unit_range(n_units, rank, world_size):
  """Half-open range [lo, hi) of flattened (b, h) units owned by `rank`; sizes differ by <= 1."""
  if not (0 <= rank < world_size):
    raise ValueError("rank out of range")
  base, extra = divmod(n_units, world_size)
  lo = rank * base + min(rank, extra)
  return lo, lo + base + (1 if rank < extra else 0)


def shard_bshd(t, rank, world_size):
  """Contiguous copy [1, S, n_local, D] (units folded into the head axis) of this rank's (b, h)
  units of a [B, S, H, D] tensor.  The head axis is independent of the batch axis for every
  kernel here, so folding is exact."""
  B, S, H, D = t.shape
  lo, hi = unit_range(B * H, rank, world_size)
  flat = t.permute(1, 0, 2, 3).reshape(S, B * H, D)  # unit index = b * H + h
  return flat[:, lo:hi, :].unsqueeze(0).contiguous()


def shard_bhs(t, rank, world_size):
  """This rank's rows of a per-unit tensor [B, H, ...] -> [1, n_local, ...]."""
  B, H = t.shape[0], t.shape[1]
  lo, hi = unit_range(B * H, rank, world_size)
  return t.reshape(B * H, *t.shape[2:])[lo:hi].unsqueeze(0).contiguous()


def gather_units(parts, B, H):
  """Inverse of shard_bhs for validation: list of [1, n_local, ...] (rank order) -> [B, H, ...]."""
  import torch
  cat = torch.cat([p.squeeze(0) for p in parts], dim=0)
  return cat.reshape(B, H, *cat.shape[1:])
