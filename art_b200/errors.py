"""HTTP-mappable errors raised by the backend (parity: reference ``src/art/errors.py:10-64``)."""
from fastapi import HTTPException


class _StatusError(HTTPException):
    status: int = 500

    def __init__(self, message: str):
        super().__init__(status_code=self.status, detail=message)


class ForbiddenBucketCreationError(_StatusError):
    """403: the bucket exists under another owner, or the credentials may not create buckets."""
    status = 403


class UnsupportedLoRADeploymentProviderError(_StatusError):
    """400: the provider has no serverless LoRA deployment."""
    status = 400


class UnsupportedBaseModelDeploymentError(_StatusError):
    """400: the provider cannot serve LoRAs for this base model."""
    status = 400


class LoRADeploymentTimedOutError(_StatusError):
    """504: the deployment job did not finish in time."""
    status = 504
