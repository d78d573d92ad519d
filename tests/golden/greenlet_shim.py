"""A stand-in for the ``greenlet`` package, enough for the reference simulator.

The reference runs the work-items (and subgroups) of a work-group as greenlets
and implements ``group.barrier()`` by switching from one to the next
(python/hckernel/kernel_api.py:378-431).  The package is not installed where
the golden vectors are generated, so this module provides the three things the
simulator uses - ``greenlet(fn)``, ``.switch()`` and the return to the parent
when a greenlet's function ends - with one thread per greenlet and a baton
that exactly one of them holds at a time.  Execution is therefore as
sequential and as deterministic as with the real package.

Used only by ``make_golden.py``; the tests read the generated files.
"""

import threading


class greenlet:  # noqa: N801  (the name the reference imports)
    _current = threading.local()

    def __init__(self, run):
        self._run = run
        self._go = threading.Semaphore(0)
        self._thread = None
        self._done = False
        self.parent = greenlet._here()
        self._error = None

    @staticmethod
    def _here():
        me = getattr(greenlet._current, "value", None)
        if me is None:  # the thread that never was a greenlet: the root
            me = greenlet._current.value = _Root()
        return me

    def _body(self):
        greenlet._current.value = self
        self._go.acquire()
        try:
            self._run()
        except BaseException as error:  # handed to the parent, like the real package
            self._error = error
        self._done = True
        self.parent._go.release()  # the function ended: back to the parent

    def switch(self):
        """Hand the baton to this greenlet; returns when someone hands it back
        to the caller (or, for a parent, when the greenlet's function ends)."""
        if self._done:
            return
        me = greenlet._here()
        if self._thread is None:
            self._thread = threading.Thread(target=self._body, daemon=True)
            self._thread.start()
        self._go.release()
        me._go.acquire()
        if isinstance(me, _Root) or True:
            error, self._error = self._error, None
            if error is not None:
                raise error


class _Root:
    def __init__(self):
        self._go = threading.Semaphore(0)
        self._error = None
