// Library-wide entry points: version, device facts, tunables, the device status word.
#include <stdlib.h>

#include "btb_b200_internal.h"
#include "../../include/btb_b200.h"

static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v != nullptr && *v != '\0') ? atoi(v) : dflt;
}

B2Tuning& b2_tuning() {
    static B2Tuning t = {
        env_int("BTB_B200_RING_BYTES", 96 * 1024), env_int("BTB_B200_SEG_BYTES", 4096),
        env_int("BTB_B200_X_SMEM_MAX", 160 * 1024), env_int("BTB_B200_CTAS_PER_SM", 1),
        env_int("BTB_B200_EVICT_FIRST", 1),        env_int("BTB_B200_PDL", 5),
        env_int("BTB_B200_WARPS", 16),             env_int("BTB_B200_SOLO", 1),
        env_int("BTB_B200_MOE_STREAM", 1),         env_int("BTB_B200_MS_TPR", 0),             env_int("BTB_B200_MS_CTAS", 0),
        env_int("BTB_B200_MS_SEG", 0),
        env_int("BTB_B200_MS_WARPS", 0),           env_int("BTB_B200_TC_STAGES", 0),
        env_int("BTB_B200_TC_CTAS", 0),
        env_int("BTB_B200_BALANCE", 1),
        env_int("BTB_B200_X_DIRECT", 1),
        env_int("BTB_B200_L2_WARM_KB", 0),         env_int("BTB_B200_L2_WARM_CTAS", 0),
        env_int("BTB_B200_WARPS_PACKED", 24),
        env_int("BTB_B200_TC_FOLD", 0),
    };
    return t;
}

int b2_sm_count() {
    static int sms[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

extern "C" int btb_b200_version(void) { return 1; }

extern "C" int btb_b200_sm_count(void) { return b2_sm_count(); }

extern "C" int btb_b200_set_tuning(const char* key, int value) {
    if (key == nullptr) return B2_ERR_NULL;
    B2Tuning& t = b2_tuning();
    if (!strcmp(key, "ring_bytes")) t.ring_bytes = value;
    else if (!strcmp(key, "seg_bytes")) t.seg_bytes = value;
    else if (!strcmp(key, "x_smem_max")) t.x_smem_max = value;
    else if (!strcmp(key, "ctas_per_sm")) t.ctas_per_sm = value;
    else if (!strcmp(key, "evict_first")) t.evict_first = value;
    else if (!strcmp(key, "pdl")) t.pdl = value;
    else if (!strcmp(key, "warps")) t.warps = value == 16 ? 16 : 8;
    else if (!strcmp(key, "balance")) t.balance = value != 0;
    else if (!strcmp(key, "solo")) t.solo = value != 0;
    else if (!strcmp(key, "moe_stream")) t.moe_stream = value != 0;
    else if (!strcmp(key, "x_direct")) t.x_direct = value != 0;
    else if (!strcmp(key, "l2_warm_kb")) t.l2_warm_kb = value < 0 ? 0 : value;
    else if (!strcmp(key, "l2_warm_ctas")) t.l2_warm_ctas = value < 0 ? 0 : value;
    else if (!strcmp(key, "warps_packed")) t.warps_packed = value;
    else if (!strcmp(key, "tc_fold")) t.tc_fold = value != 0;
    else if (!strcmp(key, "ms_tpr")) t.ms_tpr = value;
    else if (!strcmp(key, "ms_ctas")) t.ms_ctas = value < 0 ? 0 : value;
    else if (!strcmp(key, "ms_seg")) t.ms_seg = value < 0 ? 0 : value & ~31;
    else if (!strcmp(key, "ms_warps")) t.ms_warps = value < 0 ? 0 : value;
    else return B2_ERR_DOMAIN;
    return B2_OK;
}

int b2_status_take_gemv(int*);
int b2_status_take_layer(int*);
int b2_status_take_attn(int*);
int b2_status_take_step(int*);
int b2_status_take_moe(int*);
int b2_status_take_sample(int*);
int b2_status_take_moes(int*);
int b2_status_take_attno(int*);
int b2_status_take_tc(int*);
int b2_status_take_tp(int*);

extern "C" int btb_b200_status(int* code) {
    if (code == nullptr) return B2_ERR_NULL;
    int (*const take[])(int*) = {b2_status_take_gemv, b2_status_take_layer, b2_status_take_attn, b2_status_take_step,
                                 b2_status_take_moe, b2_status_take_sample, b2_status_take_moes, b2_status_take_attno, b2_status_take_tc, b2_status_take_tp};
    *code = 0;
    for (auto f : take) {
        int v = 0;
        const int rc = f(&v);
        if (rc) return rc;
        if (v != 0 && *code == 0) *code = v;
    }
    return B2_OK;
}
