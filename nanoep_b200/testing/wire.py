"""Independent restatement of the window byte layout, for tests.

Deliberately does not import the native layout code: the tests compare this arithmetic with what the
extension reports (the reference does the same with nano_ep/testing/wire.py:4-25 for its own layout).
"""


def align(value: int, to: int) -> int:
    return (value + to - 1) // to * to


def wire_row_bytes(hidden: int, topk: int) -> int:
    """bf16 x[H] then fp32 weights[K], padded to a 16-byte multiple."""
    return align(2 * hidden + 4 * topk, 16)


def wire_weights_offset(hidden: int) -> int:
    return 2 * hidden


def count_message_ints(local_experts: int) -> int:
    return 2 + local_experts


def window_regions(ranks: int, max_tokens: int, hidden: int, topk: int, num_experts: int, per_rank_reduction: bool = False) -> dict:
    local = num_experts // ranks
    region = 256
    at = 0

    def take(nbytes):
        nonlocal at
        here = at
        at = align(at + nbytes, region)
        return here

    out = {}
    out["signal_offset"] = take(32 * 8)
    out["data_signal_offset"] = take(32 * 8)
    chunks = (max_tokens + 31) // 32  # rows are planned per chunk of 32 source tokens
    ctrl_ints = 16 + (ranks + num_experts) + ranks + local + (ranks + 1) + (local + 1) + local + ranks + ranks * chunks
    out["ctrl_offset"] = take(ctrl_ints * 4)
    out["counts_in_stride"] = align(ranks * count_message_ints(local) * 4, region)
    out["counts_in_offset"] = take(2 * out["counts_in_stride"])
    out["routing_in_stride"] = align(ranks * max_tokens * topk * 4, region)
    out["routing_in_offset"] = take(2 * out["routing_in_stride"])
    out["chunks_in_stride"] = align(ranks * chunks * 4, region)
    out["chunks_in_offset"] = take(2 * out["chunks_in_stride"])
    out["stage_rows_stride"] = align(max_tokens * wire_row_bytes(hidden, topk), region)
    out["stage_rows_offset"] = take(2 * out["stage_rows_stride"])
    # return area: one copy; P partitions of [Tmax, H] bf16, a u32 arrival flag per (partition, token), fp32 weights [Tmax, K]
    parts = min(ranks, topk) if per_rank_reduction else topk
    out["ret_parts"] = parts
    out["rank_indexed"] = int(per_rank_reduction and ranks <= topk)
    out["ret_w_offset"] = take(max_tokens * topk * 4)
    out["ret_flag_offset"] = take(parts * max_tokens * 4)
    out["ret_offset"] = take(parts * max_tokens * hidden * 2)
    out["meta_scratch_offset"] = take(ranks * max_tokens * (topk + 2) * 4)
    out["slot_scratch_offset"] = take((ranks * max_tokens * topk + local * 128) * 4)
    out["num_bytes"] = at
    out["row_bytes"] = wire_row_bytes(hidden, topk)
    out["msg_ints"] = count_message_ints(local)
    return out
