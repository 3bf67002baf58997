"""A text-only stand-in for the per-GPU service process of ``msa_b200.engine.MSAEngine`` (its ``service_main``
argument): it speaks the same queue protocol -- READY, BLOCKS, IDX_TO_DOC, report_doc_id, then one GenerateResponse per
GenerateRequest until ``None`` -- and answers every prompt with a line that shows what it received."""
from msa_b200.engine import (MEMORY_WORKER_BLOCKS, MEMORY_WORKER_IDX_TO_DOC, MEMORY_WORKER_READY, GenerateResponse,
                             ReportDocID)
from msa_b200.prefill import ProtocolConstants


def service_main(gpu_id, request_queue, response_queue, generate_config, model_config, memory_config):
    ProtocolConstants.send(response_queue, MEMORY_WORKER_READY, block=False)
    docs = ProtocolConstants.expect(request_queue, MEMORY_WORKER_BLOCKS)
    idx_to_doc = ProtocolConstants.expect(request_queue, MEMORY_WORKER_IDX_TO_DOC)
    response_queue.put(ReportDocID(gpu_id=gpu_id, pooled_doc_id_bias=len(docs)), block=False)
    chunks = sum(d.num_chunks for d in docs)
    while True:
        cmd = request_queue.get()
        if cmd is None:
            return
        texts = [f"gpu{gpu_id}|docs{len(docs)}|chunks{chunks}|known{len(idx_to_doc)}|{p}|{len(ids)}"
                 for p, ids in zip(cmd.prompts, cmd.input_ids)]
        recall = {18: [{"topk_doc_ids": [gpu_id], "score": [1.0]} for _ in cmd.prompts]} if cmd.require_recall_topk else None
        response_queue.put(GenerateResponse(msg_id=cmd.msg_id, seq_id=cmd.seq_id, gpu_id=gpu_id, generated_texts=texts,
                                            recall_topk=recall))
