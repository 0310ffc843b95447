"""What every paged-cache worker shares, whatever its architecture: the pinned staging ring that carries a step's metadata to
the device in ONE copy, the device-side wait for pending swap copies, and giving a finished sequence's blocks back.
Subclasses (worker/model.py: LlamaModel, worker/bupozen_model.py: BupozenModel) own their weights, layers and cache tensors
and set `device`, `gpu_block_manager` and `cpu_block_manager`."""
from __future__ import annotations

import itertools

import numpy as np
import torch


class PagedModelBase:
    def _init_staging(self):
        # pinned staging ring for per-step metadata (eager path): a slot is rewritten only after the H2D copy that last read it
        # has completed (event per slot), so back-to-back forward_async calls never race the copy engine
        self._stage_ring = []
        self._stage_next = 0
        self._swap_done = None          # event of swap copies enqueued on a copy stream since the last forward

    _STAGE_SLOTS = 4

    def _stage_slot(self, n: int):
        """Next slot of the persistent pinned ring, grown geometrically; waits (host side) for the copy that last used it."""
        i = self._stage_next
        self._stage_next = (i + 1) % self._STAGE_SLOTS
        if len(self._stage_ring) <= i:
            self._stage_ring.append(None)
        slot = self._stage_ring[i]
        if slot is None or slot[0].numel() < n:
            cap = max(4096, 1 << (max(n, 1) - 1).bit_length())
            if slot is not None:
                slot[1].synchronize()
            slot = (torch.empty((cap,), dtype=torch.int32).pin_memory(), torch.cuda.Event())
            self._stage_ring[i] = slot
        else:
            slot[1].synchronize()                # no-op unless the copy engine is more than _STAGE_SLOTS steps behind
        return slot

    def _wait_for_swaps(self):
        """Device-side wait (no host sync) for swap copies enqueued on the copy stream since the last forward."""
        if self._swap_done is not None and not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()):
            torch.cuda.current_stream().wait_event(self._swap_done)
            self._swap_done = None

    def _stage_metadata(self, *parts):
        """One persistent pinned host buffer (ring of slots), one async H2D copy; returns int32 device views (one per list)."""
        flat = np.fromiter(itertools.chain(*parts), dtype=np.int32)
        host, ev = self._stage_slot(flat.size)
        host[:flat.size].numpy()[:] = flat
        dev = host[:flat.size].to(self.device, non_blocking=True)
        ev.record()
        views, off = [], 0
        for p in parts:
            views.append(dev[off:off + len(p)])
            off += len(p)
        return views

    @torch.inference_mode()
    def free_seqs_resources(self, seq_ids_list: list):
        """model.py:401-408."""
        seq_ids = torch.tensor(seq_ids_list, dtype=torch.int32, device=self.device)
        self.gpu_block_manager.free_blocks_for_seqs(seq_ids, seq_ids_list=seq_ids_list)
        self.cpu_block_manager.free_blocks_for_seqs(seq_ids, seq_ids_list=seq_ids_list)
