// Placeholder until the transfer engine lands: a store server needs no extra bookkeeping without it.
#include "mf_api_internal.h"
namespace mf {
namespace api {
void AttachTransFaultHandler(store::StoreServer *) {}
}  // namespace api
}  // namespace mf
