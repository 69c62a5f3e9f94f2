/* voxtral_b200_dropin.h - state shared by the two replacement translation units. */
#ifndef VOXTRAL_B200_DROPIN_H
#define VOXTRAL_B200_DROPIN_H

#include <stdint.h>

/* The frame tts_llm_forward has already computed for the tts_acoustic_forward call
 * that follows it in the orchestrator's loop (voxtral_tts.c:302-305). */
typedef struct {
    int valid;
    float hidden[3072];
    int codes[37];
    uint64_t rng_before, rng_after;
} vb200_pending_frame_t;

extern vb200_pending_frame_t vb200_pending;

#endif
