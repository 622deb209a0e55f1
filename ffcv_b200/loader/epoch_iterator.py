"""Asynchronous batch pump of one epoch (reference: ``ffcv/loader/epoch_iterator.py:33-176``).

Same structure as the reference: a worker thread walks the batches, each batch uses one slot of a
ring of ``batches_ahead + 2`` buffer sets with its own CUDA stream, results travel through a
bounded queue, the consumer's stream waits on the slot's stream in ``__next__``, and a slot is
only refilled after an event recorded on the consumer's stream says the batch that used it
before has been consumed.  Three differences: what runs on the slot's stream is the native
decode-and-augment call instead of a host->device copy of decoded pixels; the "consumed" event
of a batch is recorded when the consumer asks for the next batch (the reference records it at
hand-over time, which chains every new batch behind the consumer's latest work and keeps copies
from overlapping compute); and an exception in the worker is handed to the consumer and re-raised
there instead of leaving it blocked.
"""
from queue import Full, Queue
from threading import Event, Thread
from typing import Sequence

import numpy as np
import torch as ch


class _Failure:
    def __init__(self, exc):
        self.exc = exc


class EpochIterator(Thread):
    def __init__(self, loader, order: Sequence[int], epoch: int):
        super().__init__(daemon=True)
        self.loader = loader
        self.order = np.asarray(order)
        self.epoch = epoch
        bs = loader.batch_size
        self.batches = [self.order[i:i + bs] for i in range(0, len(self.order), bs)]
        self.slots = loader.batches_ahead + 2
        self.output_queue = Queue(loader.batches_ahead)
        self.terminate_event = Event()
        self.closed = False
        self.memory_context = loader.memory_manager.schedule_epoch(self.batches)
        self.memory_context.__enter__()
        self.storage_state = self.memory_context.state
        self.is_cuda = ch.cuda.is_available()
        self.device = loader.device
        if self.is_cuda:
            self.current_stream = ch.cuda.current_stream(self.device)
            self.cuda_streams = loader.slot_streams()
        else:
            self.current_stream = None
            self.cuda_streams = [None] * self.slots
        self.buffers = loader.slot_buffers()
        self.slot_done = loader.slot_done_events()
        # consumed[s]: recorded on the consumer's stream once the consumer has moved past the batch
        # that used slot s, i.e. when it asks for the following batch.  The queue bound guarantees
        # the worker reaches a slot again only after that (it can run batches_ahead + 1 batches
        # ahead of the batch being consumed and the ring has batches_ahead + 2 slots).  Output
        # buffers live across epochs, so every slot first waits for what the consumer had queued
        # when this epoch started.
        start_event = None
        if self.is_cuda:
            start_event = ch.cuda.Event()
            start_event.record(self.current_stream)
        self.consumed = [start_event] * self.slots
        self.last_slot = None
        self.start()

    def run(self):
        slot = 0
        try:
            if self.is_cuda:
                ch.cuda.set_device(self.device)
            for b_ix, ixes in enumerate(self.batches):
                if self.terminate_event.is_set():
                    return
                result = self.run_pipeline(b_ix, ixes, slot, self.consumed[slot])
                item = (slot, result)
                while True:
                    try:
                        self.output_queue.put(item, block=True, timeout=0.5)
                        break
                    except Full:
                        pass
                    if self.terminate_event.is_set():
                        return
                slot = (slot + 1) % self.slots
            self.output_queue.put(None)
        except BaseException as exc:  # noqa: BLE001 - forwarded to the consumer
            self.output_queue.put(_Failure(exc))

    def run_pipeline(self, b_ix, batch_indices, slot, cuda_event):
        self.memory_context.start_batch(b_ix)
        stream = self.cuda_streams[slot]
        if not self.is_cuda:
            return self.loader.graph.run_batch(batch_indices, slot, None, self.buffers, self.storage_state,
                                               self.epoch, b_ix)
        # The slot's pinned staging buffer is about to be rewritten by the host: the copy and the
        # kernels of the batch that used it last must have finished (a host-side wait; that batch
        # was queued batches_ahead + 2 batches ago).
        if self.slot_done[slot] is not None:
            self.slot_done[slot].synchronize()
        with ch.cuda.stream(stream):
            if cuda_event is not None:
                cuda_event.wait()
            lookahead = self.batches[b_ix + 1] if b_ix + 1 < len(self.batches) else None
            result = self.loader.graph.run_batch(batch_indices, slot, stream.cuda_stream, self.buffers,
                                                 self.storage_state, self.epoch, b_ix, lookahead=lookahead)
            done = ch.cuda.Event()
            done.record(stream)
            self.slot_done[slot] = done
            return result

    def __next__(self):
        if self.is_cuda and self.last_slot is not None:
            event = ch.cuda.Event()
            event.record(self.current_stream)
            self.consumed[self.last_slot] = event
            self.last_slot = None
        item = self.output_queue.get()
        if item is None:
            self.close()
            raise StopIteration()
        if isinstance(item, _Failure):
            self.close()
            raise item.exc
        slot, result = item
        if self.is_cuda:
            self.current_stream.wait_stream(self.cuda_streams[slot])
            self.last_slot = slot
        return result

    def __iter__(self):
        return self

    def retire(self):
        """Stops the worker (it finishes the batch it is on) and waits for it: the slot ring is
        shared by the epochs of a loader, so two workers must never run at once."""
        self.close()
        if self.is_alive():
            self.join()

    def close(self):
        self.terminate_event.set()
        if not self.closed:
            self.closed = True
            self.memory_context.__exit__(None, None, None)

    def __del__(self):
        self.close()
