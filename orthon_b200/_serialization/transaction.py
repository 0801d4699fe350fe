"""Restore transaction: recipients are prepared in order (model first, then the optimizer, which
is told where the model's parameters will live), nothing live is touched until every recipient
has prepared, then they commit in the same order with reverse rollback on failure.
(reference project: python/orthon/_serialization/transaction.py:23-84)"""
from .._state import PreparedLoad, commit_prepared
from .format import fail


def generic_participant(owner, state, map_location):
    """Duck-typed recipient: snapshot its public state, restore through load_state_dict."""
    import copy
    before = copy.copy(owner.state_dict())

    def commit():
        try:
            owner.load_state_dict(state, map_location=map_location)
        except TypeError:
            owner.load_state_dict(state)

    def rollback():
        owner.load_state_dict(before)

    return PreparedLoad(commit, rollback)


class RestoreTransaction:
    def __init__(self, map_location=None):
        self._map_location = map_location
        self._participants = []
        self._placement = None
        self._committed = False

    def prepare_model(self, model, state):
        if state is None:
            fail("checkpoint has no model section")
        prep = getattr(model, "_prepare_load_state_dict", None)
        part = prep(state, map_location=self._map_location) if prep is not None else generic_participant(
            model, state, self._map_location)
        self._placement = part.placement  # the optimizer adopts the model's future placement
        self._participants.append(part)
        return self

    def prepare_optimizer(self, optimizer, state):
        if state is None:
            fail("checkpoint has no optimizer section")
        prep = getattr(optimizer, "_prepare_load_state_dict", None)
        if prep is not None:
            self._participants.append(prep(state, map_location=self._map_location, placement=self._placement))
        else:
            self._participants.append(generic_participant(optimizer, state, self._map_location))
        return self

    @classmethod
    def prepare(cls, model, model_state, optimizer, optimizer_state, map_location=None):
        tx = cls(map_location)
        if model is not None:
            tx.prepare_model(model, model_state)
        if optimizer is not None:
            tx.prepare_optimizer(optimizer, optimizer_state)
        return tx

    def commit(self):
        if self._committed:
            raise RuntimeError("checkpoint: restore transaction was already committed")
        self._committed = True
        commit_prepared(self._participants)
