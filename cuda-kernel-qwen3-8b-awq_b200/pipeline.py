"""One process per GPU: wiring of the layer-pipeline ring over torch.distributed.

The reference splits its 36 layers over exactly two GPUs inside one process (Inference.cu:43-47,
376-378).  Here every rank owns one stage (rank r runs the layers qw3_stage_layers gives it, the
embedding lives on rank 0, final norm + unembed + arg-max on the last rank).  torch.distributed is
only the plumbing that exchanges the 64-byte CUDA IPC handles of the stages' mailboxes; the data
path itself is peer stores over NVLink issued by the engine's own kernels, no collective.  The same
plumbing serves the row-split mode (connect_all), where every rank runs all layers on its share of
every matrix and the partial sums cross NVLink inside the pass kernel.
"""
import ctypes as C

from . import cabi


def ring_neighbours(rank, world):
    """(next, previous) stage of `rank` in the ring 0 -> 1 -> ... -> world-1 -> 0."""
    return (rank + 1) % world, (rank - 1) % world


def stage_layers(config, stage):
    """(first_layer, n_layers) of a stage: the reference's 18/18 split generalised to 1..8 stages
    (36 layers on 8 stages: 5,5,5,5,4,4,4,4)."""
    first, count = C.c_int32(0), C.c_int32(0)
    cabi.check(cabi.lib().qw3_stage_layers(C.byref(config), stage, C.byref(first), C.byref(count)), "qw3_stage_layers")
    return first.value, count.value


def exchange_handles(my_handle_bytes, dist, group=None):
    """All-gather of the 64-byte handles; returns the list indexed by rank."""
    world = dist.get_world_size(group)
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(my_handle_bytes), group=group)
    return gathered


def connect_ring(infer, dist, group=None):
    """Exchange mailbox handles and map the ring neighbours' mailboxes into this process."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    buf = (C.c_uint8 * 64)()
    cabi.check(cabi.lib().qw3_stage_export(infer._h, buf), "qw3_stage_export")
    handles = exchange_handles(bytes(buf), dist, group)
    nxt, prv = ring_neighbours(rank, world)
    hn = (C.c_uint8 * 64).from_buffer_copy(handles[nxt])
    hp = (C.c_uint8 * 64).from_buffer_copy(handles[prv])
    cabi.check(cabi.lib().qw3_stage_connect(infer._h, hn, hp), "qw3_stage_connect")


def connect_all(infer, dist, group=None):
    """Row-split tensor parallelism: exchange the handles of the ranks' exchange buffers and map every peer's."""
    world = dist.get_world_size(group)
    buf = (C.c_uint8 * 64)()
    cabi.check(cabi.lib().qw3_tp_export(infer._h, buf), "qw3_tp_export")
    handles = exchange_handles(bytes(buf), dist, group)
    flat = (C.c_uint8 * (64 * world)).from_buffer_copy(b"".join(handles))
    cabi.check(cabi.lib().qw3_tp_connect(infer._h, flat), "qw3_tp_connect")
    dist.barrier(group)   # nobody generates before every rank has mapped every buffer


def broadcast_ids(ids, n, dist, group=None):
    """The generated ids come out of the last stage's process: give them to every rank."""
    world = dist.get_world_size(group)
    box = [list(ids) if dist.get_rank(group) == world - 1 else None]
    dist.broadcast_object_list(box, src=world - 1, group=group)
    return box[0][:n]
