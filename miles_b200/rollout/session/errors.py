"""Errors of the session server and the HTTP status each maps to:

    SessionError                       500
    |- SessionNotFoundError            404  the session id is unknown
    |- MessageValidationError          400  the conversation does not extend the session (or is malformed)
    |- TruncatedGenerationError        409  a request extends a generation that ended at the length limit
    |- TokenizationError               500  the token-in-token-out invariant broke (prefix mismatch)
    `- UpstreamResponseError           502  the engine's answer is unusable

Reference: miles/rollout/session/errors.py:1-60.
"""


class SessionError(Exception):
    status_code = 500


class SessionNotFoundError(SessionError):
    status_code = 404


class MessageValidationError(SessionError, ValueError):
    status_code = 400


class TruncatedGenerationError(SessionError, ValueError):
    status_code = 409


class TokenizationError(SessionError):
    status_code = 500


class UpstreamResponseError(SessionError):
    status_code = 502
