"""Data-parallel sharding of independent basecall chunks: rank r of `world` owns a contiguous
slice of the chunk (batch) axis; weights, tables and scales are replicated. There is no
collective on the data path -- results are only concatenated."""


def shard_range(n_items, rank, world):
    """[begin, end) of the items owned by `rank`; slice lengths differ by at most one."""
    base, extra = divmod(n_items, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_chunks(x, rank, world, dim):
    """The slice of tensor `x` along `dim` owned by `rank` (a view)."""
    b, e = shard_range(x.size(dim), rank, world)
    return x.narrow(dim, b, e - b)
