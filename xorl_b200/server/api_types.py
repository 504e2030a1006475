"""Wire types of the REST training API (Tinker-compatible), cf.
src/xorl/server/api_server/api_types.py:38-1254."""
from __future__ import annotations

from typing import Any, Dict, List, Literal, Optional, Union

from pydantic import BaseModel, Field


class TensorData(BaseModel):
    data: List[Any]
    dtype: str = "int64"
    shape: Optional[List[int]] = None

    def to_list(self) -> List[Any]:
        return self.data


class ModelInput(BaseModel):
    tokens: Optional[List[int]] = None
    chunks: Optional[List[Dict[str, Any]]] = None

    def token_ids(self) -> List[int]:
        if self.tokens is not None:
            return list(self.tokens)
        out: List[int] = []
        for c in self.chunks or []:
            out += list(c.get("tokens", []))
        return out


class Datum(BaseModel):
    """One training example: the input tokens plus per-token loss inputs
    (``target_tokens``/``weights`` for cross-entropy, ``logprobs``/``advantages`` for RL losses)."""
    model_input: ModelInput
    loss_fn_inputs: Dict[str, TensorData] = Field(default_factory=dict)


class AdamParams(BaseModel):
    learning_rate: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-12
    weight_decay: float = 0.0


class ForwardBackwardInput(BaseModel):
    data: List[Datum]
    loss_fn: str = "cross_entropy"
    loss_fn_config: Dict[str, Any] = Field(default_factory=dict)


class ForwardBackwardRequest(BaseModel):
    model_id: str = "default"
    seq_id: Optional[int] = None
    forward_backward_input: ForwardBackwardInput


class ForwardRequest(BaseModel):
    model_id: str = "default"
    seq_id: Optional[int] = None
    forward_input: ForwardBackwardInput


class OptimStepRequest(BaseModel):
    model_id: str = "default"
    seq_id: Optional[int] = None
    adam_params: AdamParams = Field(default_factory=AdamParams)
    gradient_clip: Optional[float] = None


class AbortGradientEpochRequest(BaseModel):
    model_id: str = "default"


class UntypedAPIFuture(BaseModel):
    request_id: str
    model_id: Optional[str] = None


class FutureRetrieveRequest(BaseModel):
    request_id: str


class TryAgainResponse(BaseModel):
    type: Literal["try_again"] = "try_again"
    request_id: str
    queue_state: str = "active"


class RequestFailedResponse(BaseModel):
    type: Literal["request_failed"] = "request_failed"
    request_id: str
    error: str
    category: str = "server"


class CreateModelRequest(BaseModel):
    model_id: Optional[str] = None
    base_model: Optional[str] = None
    lora_config: Optional[Dict[str, Any]] = None
    session_id: Optional[str] = None


class UnloadModelRequest(BaseModel):
    model_id: str


class CreateSessionRequest(BaseModel):
    tags: List[str] = Field(default_factory=list)
    user_metadata: Dict[str, Any] = Field(default_factory=dict)


class SessionHeartbeatRequest(BaseModel):
    session_id: str


class SaveWeightsRequest(BaseModel):
    model_id: str = "default"
    path: Optional[str] = None
    seq_id: Optional[int] = None


class LoadWeightsRequest(BaseModel):
    model_id: str = "default"
    path: str
    load_optimizer: bool = True


class DeleteCheckpointRequest(BaseModel):
    model_id: str = "default"
    name: str


class InferenceEndpoint(BaseModel):
    url: str
    world_size: int = 1
    name: Optional[str] = None


class SyncWeightsRequest(BaseModel):
    model_id: str = "default"
    backend: Literal["nccl_broadcast", "peer_copy", "sparse_delta", "file"] = "nccl_broadcast"
    quantization: Optional[str] = None
    bucket_size_mb: Optional[int] = None            # None: the server's sync_bucket_size_mb


class SetSyncQuantizationRequest(BaseModel):
    format: Optional[Literal["fp8", "nvfp4", "bf16"]] = None


class ForwardBackwardOutput(BaseModel):
    loss_fn_output_type: str = "scalar"
    loss_fn_outputs: List[Dict[str, TensorData]] = Field(default_factory=list)
    metrics: Dict[str, float] = Field(default_factory=dict)


class OptimStepResponse(BaseModel):
    metrics: Dict[str, float] = Field(default_factory=dict)
