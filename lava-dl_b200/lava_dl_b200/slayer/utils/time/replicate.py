"""Replication of a tensor along a new time axis
(``src/lava/lib/dl/slayer/utils/time/replicate.py:10-37``)."""


def replicate(input, num_steps):
    """Repeat ``input`` ``num_steps`` times along a new last (time) dimension.

    The reference does this with ``F.interpolate(..., mode='nearest')`` on the tensor with a
    trailing axis of length one, which accepts inputs of 2 to 4 dimensions; the same
    values (and the same gradient, the sum over time) come from a broadcast.

    Parameters
    ----------
    input : torch tensor
    num_steps : int

    Returns
    -------
    torch tensor of shape ``input.shape + (num_steps,)``
    """
    if not 2 <= input.dim() <= 4:
        raise NotImplementedError(
            f'Input Error: Only 3D, 4D and 5D input Tensors supported (got {input.dim() + 1}D) '
            f'for the modes: nearest')
    return input.unsqueeze(-1).expand(*input.shape, int(num_steps)).contiguous()
