"""Exception hierarchy (same public names as the reference's src/olmo_core/exceptions.py)."""

__all__ = [
    "OLMoError",
    "OLMoInvalidRangeRequestError",
    "OLMoNetworkError",
    "OLMoEnvironmentError",
    "OLMoUserError",
    "OLMoCheckpointError",
    "OLMoConfigurationError",
    "OLMoCLIError",
    "OLMoThreadError",
    "OLMoUploadError",
    "OLMoDistributedTimeoutError",
    "BeakerInsufficientResourcesError",
    "OLMoBeakerExperimentFailedError",
]


class OLMoError(Exception):
    """Root of every error raised on purpose by the framework."""


class OLMoInvalidRangeRequestError(OLMoError):
    """A ranged read asked for bytes outside of the object."""


class OLMoNetworkError(OLMoError):
    """A remote storage or HTTP request failed after retries."""


class OLMoEnvironmentError(OLMoError):
    """The process environment (env vars, devices, launch mode) is not what the code needs."""


class OLMoUserError(OLMoError):
    """The caller used an API incorrectly."""


class OLMoCheckpointError(OLMoError):
    """A checkpoint is missing, incomplete or inconsistent with the model."""


class OLMoConfigurationError(OLMoError):
    """A configuration object holds an invalid or contradictory value."""


class OLMoCLIError(OLMoError):
    """Bad command-line usage."""


class OLMoThreadError(OLMoError):
    """A background thread died."""


class OLMoUploadError(OLMoError):
    """Uploading a file to remote storage failed."""


class OLMoDistributedTimeoutError(OLMoError):
    """A bounded device-side or host-side wait on another rank expired."""


class BeakerInsufficientResourcesError(OLMoError):
    """Kept for API parity with launch tooling."""


class OLMoBeakerExperimentFailedError(OLMoError):
    """Kept for API parity with launch tooling."""
