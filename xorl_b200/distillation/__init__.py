"""On-policy distillation support: teacher log-probability stores and the glue that fills them
(cf. src/xorl/distillation/)."""
from .teacher_store import TeacherLogprobStore, attach_teacher_logprobs, score_with_teacher  # noqa: F401
