#pragma once
namespace llis { namespace job { class FinishedBlockNotifier; } }
