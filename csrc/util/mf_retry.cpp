#include "mf_retry.h"

namespace mf {

RetryPolicy &GlobalRetryPolicy()
{
    static RetryPolicy p;
    return p;
}

RetryStats &GlobalRetryStats()
{
    static RetryStats s;
    return s;
}

}  // namespace mf
