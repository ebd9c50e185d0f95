"""Failure classes of the OCS (optical circuit switch) runtime
(reference: pccl/ocs/exceptions.py:4-21)."""


class OCSError(RuntimeError):
    """Any OCS runtime failure."""


class OCSPlanMismatchError(OCSError):
    """Ranks reached one barrier holding different plans."""


class OCSBarrierTimeout(OCSError):
    """A participant's READY never arrived."""


class OCSLinkNotReady(OCSError):
    """The switch finished but the links did not report alignment."""


class OCSProtocolError(OCSError):
    """A control-plane wire message failed validation."""
