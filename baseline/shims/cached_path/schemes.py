"""Scheme-client registry stand-in: the reference registers its own clients at import time."""

_CLIENTS = []


class SchemeClient:
    recoverable_errors = (ConnectionError, TimeoutError)
    scheme = ""

    def __init__(self, resource: str):
        self.resource = resource


class S3Client(SchemeClient):
    scheme = "s3"


def add_scheme_client(client) -> None:
    _CLIENTS.append(client)
